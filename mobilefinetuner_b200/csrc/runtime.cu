// Runtime part of libmft_cuda.so: initialisation, error reporting, the caching
// device allocator (the device analogue of the reference's MemoryManager /
// MemoryPool, operator/finetune_ops/core/memory_manager.cpp:34-145) and copies.
#include <cstdlib>
#include <atomic>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace mft {

static thread_local std::string g_last_error;
static std::atomic<int64_t> g_launches{0};
static int32_t* g_status_word = nullptr;
static int g_device = -1;
static std::mutex g_init_mutex;

void set_error(const std::string& msg) { g_last_error = msg; }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
bool dep_launch_enabled() {
    static const bool on = [] { const char* e = std::getenv("MFT_PDL"); return e ? std::atoi(e) != 0 : false; }();
    return on;
}
int32_t* device_status_word() { return g_status_word; }

int32_t fail(int32_t code, const std::string& msg) {
    set_error(msg);
    return code;
}
int32_t check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return MFT_OK;
    set_error(std::string(what) + ": " + cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? MFT_ERR_OOM : MFT_ERR_CUDA;
}

// ---- caching allocator ------------------------------------------------------
// Blocks are rounded up to a size class (512 B granularity below 1 MiB, 2 MiB
// granularity above) and kept in per-class free lists when released.  Lookup of
// a live pointer is a hash probe, not the reference's linear scan.
struct Allocator {
    std::mutex mu;
    std::unordered_map<void*, size_t> live;             // ptr -> rounded size
    std::map<size_t, std::vector<void*>> free_lists;    // rounded size -> cached blocks
    int64_t in_use = 0, cached = 0, peak = 0, n_cuda_malloc = 0;

    static size_t round_size(size_t b) {
        if (b == 0) b = 1;
        const size_t small = 512, big = size_t(2) << 20;
        if (b < (size_t(1) << 20)) return (b + small - 1) / small * small;
        return (b + big - 1) / big * big;
    }
    int32_t alloc(size_t bytes, void** out) {
        const size_t sz = round_size(bytes);
        std::lock_guard<std::mutex> lk(mu);
        auto it = free_lists.find(sz);
        void* p = nullptr;
        if (it != free_lists.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
            cached -= (int64_t)sz;
        } else {
            cudaError_t e = cudaMalloc(&p, sz);
            if (e != cudaSuccess) {
                cudaGetLastError();
                release_cached_locked();
                e = cudaMalloc(&p, sz);
                if (e != cudaSuccess) {
                    cudaGetLastError();
                    return fail(MFT_ERR_OOM, "mft_malloc: out of device memory");
                }
            }
            ++n_cuda_malloc;
        }
        live[p] = sz;
        in_use += (int64_t)sz;
        if (in_use > peak) peak = in_use;
        *out = p;
        return MFT_OK;
    }
    int32_t release(void* p) {
        if (!p) return MFT_OK;
        std::lock_guard<std::mutex> lk(mu);
        auto it = live.find(p);
        if (it == live.end()) return fail(MFT_ERR_INVALID_ARG, "mft_free: unknown pointer");
        const size_t sz = it->second;
        live.erase(it);
        free_lists[sz].push_back(p);
        in_use -= (int64_t)sz;
        cached += (int64_t)sz;
        return MFT_OK;
    }
    void release_cached_locked() {
        for (auto& kv : free_lists)
            for (void* p : kv.second) cudaFree(p);
        free_lists.clear();
        cached = 0;
    }
};
static Allocator g_alloc;

}  // namespace mft

using namespace mft;

extern "C" {

int32_t mft_init(int32_t device) {
    std::lock_guard<std::mutex> lk(g_init_mutex);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(MFT_ERR_CUDA, "mft_init: no CUDA device available (this library has no CPU fallback)");
    }
    if (device < 0 || device >= n) return fail(MFT_ERR_INVALID_ARG, "mft_init: bad device index");
    if (int32_t s = check_cuda(cudaSetDevice(device), "cudaSetDevice")) return s;
    if (g_device == device && g_status_word) return MFT_OK;
    cudaDeviceProp prop;
    if (int32_t s = check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return s;
    if (prop.major != 10)
        return fail(MFT_ERR_UNSUPPORTED, "mft_init: kernels are built for sm_100a only; found sm_" +
                                             std::to_string(prop.major) + std::to_string(prop.minor));
    g_device = device;
    if (int32_t s = check_cuda(cudaMalloc(&g_status_word, 256), "cudaMalloc(status)")) return s;
    if (int32_t s = check_cuda(cudaMemset(g_status_word, 0, 256), "cudaMemset(status)")) return s;
    return MFT_OK;
}

int32_t mft_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_init_mutex);
    {
        std::lock_guard<std::mutex> lk2(g_alloc.mu);
        g_alloc.release_cached_locked();
    }
    if (g_status_word) {
        cudaFree(g_status_word);
        g_status_word = nullptr;
    }
    g_device = -1;
    return MFT_OK;
}

const char* mft_last_error(void) { return g_last_error.c_str(); }
int32_t mft_version(void) { return 100; }
int64_t mft_launch_count(void) { return g_launches.load(); }
void mft_launch_count_reset(void) { g_launches.store(0); }

int32_t mft_stream_sync(mft_stream_t stream) {
    return check_cuda(cudaStreamSynchronize(as_stream(stream)), "cudaStreamSynchronize");
}

int32_t mft_device_status(mft_stream_t stream, int32_t* status_host) {
    if (!g_status_word) return fail(MFT_ERR_INVALID_ARG, "mft_device_status: call mft_init first");
    int32_t v = 0;
    if (int32_t s = check_cuda(cudaMemcpyAsync(&v, g_status_word, 4, cudaMemcpyDeviceToHost, as_stream(stream)), "status copy")) return s;
    if (int32_t s = check_cuda(cudaStreamSynchronize(as_stream(stream)), "status sync")) return s;
    if (v != 0) cudaMemsetAsync(g_status_word, 0, 4, as_stream(stream));
    if (status_host) *status_host = v;
    return MFT_OK;
}

int32_t mft_malloc(size_t bytes, void** ptr) {
    MFT_CHECK_ARG(ptr != nullptr, "mft_malloc: null out pointer");
    return g_alloc.alloc(bytes, ptr);
}
int32_t mft_free(void* ptr) { return g_alloc.release(ptr); }
int32_t mft_empty_cache(void) {
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    g_alloc.release_cached_locked();
    return MFT_OK;
}
int32_t mft_mem_stats(int64_t* s) {
    MFT_CHECK_ARG(s != nullptr, "mft_mem_stats: null pointer");
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    s[0] = g_alloc.in_use; s[1] = g_alloc.cached; s[2] = g_alloc.peak; s[3] = g_alloc.n_cuda_malloc;
    return MFT_OK;
}

int32_t mft_memcpy_h2d(void* dst, const void* src, size_t bytes, mft_stream_t stream) {
    return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)), "memcpy h2d");
}
int32_t mft_memcpy_d2h(void* dst, const void* src, size_t bytes, mft_stream_t stream) {
    if (int32_t s = check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)), "memcpy d2h")) return s;
    return check_cuda(cudaStreamSynchronize(as_stream(stream)), "memcpy d2h sync");
}
int32_t mft_host_alloc(size_t bytes, void** out_host) {
    MFT_CHECK_ARG(out_host && bytes > 0, "mft_host_alloc: bad argument");
    return check_cuda(cudaHostAlloc(out_host, bytes, cudaHostAllocDefault), "pinned host allocation");
}
int32_t mft_host_free(void* host) { return host ? check_cuda(cudaFreeHost(host), "pinned host free") : MFT_OK; }
int32_t mft_memcpy_d2d(void* dst, const void* src, size_t bytes, mft_stream_t stream) {
    return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)), "memcpy d2d");
}
int32_t mft_memset(void* dst, int32_t value, size_t bytes, mft_stream_t stream) {
    return check_cuda(cudaMemsetAsync(dst, value, bytes, as_stream(stream)), "memset");
}

}  // extern "C"
