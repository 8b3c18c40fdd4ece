// Runtime part of libmft_cuda.so: initialisation, error reporting, the caching
// device allocator (the device analogue of the reference's MemoryManager /
// MemoryPool, operator/finetune_ops/core/memory_manager.cpp:34-145) and copies.
#include <cstdio>
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

namespace {
struct LaunchReport {
    std::string path;
    std::mutex mu;
    std::map<std::string, int64_t> counts;
    LaunchReport() { if (const char* e = std::getenv("MFT_LAUNCH_REPORT")) path = e; }
    ~LaunchReport() {
        if (path.empty()) return;
        if (FILE* f = std::fopen(path.c_str(), "w")) {
            for (const auto& kv : counts) std::fprintf(f, "%s %lld\n", kv.first.c_str(), (long long)kv.second);
            std::fclose(f);
        }
    }
};
LaunchReport& launch_report() { static LaunchReport r; return r; }
}  // namespace
void note_launch(const char* name) {
    LaunchReport& r = launch_report();
    if (r.path.empty()) return;
    std::lock_guard<std::mutex> lk(r.mu);
    ++r.counts[name];
}
// MFT_PDL=0 / 1 in the environment decides for the whole process; without it the caller's hint does (per host thread:
// launches are issued synchronously by the thread that runs a step).
static thread_local bool t_dep_hint = false;
bool set_dep_launch_hint(bool on) { const bool old = t_dep_hint; t_dep_hint = on; return old; }
bool dep_launch_enabled() {
    static const int mode = [] { const char* e = std::getenv("MFT_PDL"); return e ? (std::atoi(e) != 0 ? 1 : 0) : -1; }();
    return mode >= 0 ? mode != 0 : t_dep_hint;
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
//
// Stream order: mft_free(ptr, stream) promises that every use of the block was
// queued on `stream` (or made visible to it) before the call.  The block goes
// to the free list with an event recorded on that stream.  mft_malloc(bytes,
// stream) hands a cached block out at once when it was freed on the same stream
// (later work on the stream runs after the earlier uses anyway) or when its
// event has completed; otherwise the requesting stream is made to wait for the
// event, so a kernel of another stream that still reads the block finishes
// before the new owner's first write.  Nothing blocks the host.
struct Allocator {
    struct Cached {
        void* ptr;
        cudaStream_t stream;     // stream the block was released on
        cudaEvent_t done;        // recorded on that stream at release (null: released with no work pending)
    };
    std::mutex mu;
    std::unordered_map<void*, size_t> live;              // ptr -> rounded size
    std::map<size_t, std::vector<Cached>> free_lists;    // rounded size -> cached blocks
    std::vector<cudaEvent_t> event_pool;
    int64_t in_use = 0, cached = 0, peak = 0, n_cuda_malloc = 0, n_reuse = 0, n_cross_stream_waits = 0;

    static size_t round_size(size_t b) {
        if (b == 0) b = 1;
        const size_t small = 512, big = size_t(2) << 20;
        if (b < (size_t(1) << 20)) return (b + small - 1) / small * small;
        return (b + big - 1) / big * big;
    }
    cudaEvent_t take_event() {
        if (!event_pool.empty()) { cudaEvent_t e = event_pool.back(); event_pool.pop_back(); return e; }
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        return e;
    }
    int32_t alloc(size_t bytes, cudaStream_t stream, void** out) {
        const size_t sz = round_size(bytes);
        std::lock_guard<std::mutex> lk(mu);
        auto it = free_lists.find(sz);
        void* p = nullptr;
        if (it != free_lists.end() && !it->second.empty()) {
            // prefer a block whose release is already ordered before `stream`: same stream, or event complete
            std::vector<Cached>& fl = it->second;
            size_t pick = fl.size() - 1;
            for (size_t i = fl.size(); i-- > 0;) {
                if (!fl[i].done || fl[i].stream == stream) { pick = i; break; }
                if (cudaEventQuery(fl[i].done) == cudaSuccess) { pick = i; break; }
                cudaGetLastError();
            }
            Cached c = fl[pick];
            fl.erase(fl.begin() + (std::ptrdiff_t)pick);
            if (c.done) {
                if (c.stream != stream && cudaEventQuery(c.done) != cudaSuccess) {
                    cudaGetLastError();
                    if (int32_t s = check_cuda(cudaStreamWaitEvent(stream, c.done, 0), "mft_malloc: wait for the releasing stream")) {
                        fl.push_back(c);
                        return s;
                    }
                    ++n_cross_stream_waits;
                }
                event_pool.push_back(c.done);
            }
            p = c.ptr;
            cached -= (int64_t)sz;
            ++n_reuse;
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
    int32_t release(void* p, cudaStream_t stream) {
        if (!p) return MFT_OK;
        std::lock_guard<std::mutex> lk(mu);
        auto it = live.find(p);
        if (it == live.end()) return fail(MFT_ERR_INVALID_ARG, "mft_free: unknown pointer");
        const size_t sz = it->second;
        Cached c{p, stream, take_event()};
        if (c.done && cudaEventRecord(c.done, stream) != cudaSuccess) {
            // cannot order the release (e.g. the stream is being captured): fall back to a full device wait on reuse
            cudaGetLastError();
            event_pool.push_back(c.done);
            c.done = nullptr;
            cudaDeviceSynchronize();
        }
        live.erase(it);
        free_lists[sz].push_back(c);
        in_use -= (int64_t)sz;
        cached += (int64_t)sz;
        return MFT_OK;
    }
    // Frees cached blocks, largest size class first, until at most `keep_bytes` stay cached.
    void trim_locked(int64_t keep_bytes) {
        for (auto it = free_lists.rbegin(); it != free_lists.rend() && cached > keep_bytes; ++it) {
            std::vector<Cached>& fl = it->second;
            while (!fl.empty() && cached > keep_bytes) {
                Cached c = fl.back();
                fl.pop_back();
                cudaFree(c.ptr);
                if (c.done) event_pool.push_back(c.done);
                cached -= (int64_t)it->first;
            }
        }
    }
    // cudaFree waits for the device to go idle, so no event needs to be consulted here.
    void release_cached_locked() {
        for (auto& kv : free_lists)
            for (Cached& c : kv.second) {
                cudaFree(c.ptr);
                if (c.done) event_pool.push_back(c.done);
            }
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

int32_t mft_malloc(size_t bytes, mft_stream_t stream, void** ptr) {
    MFT_CHECK_ARG(ptr != nullptr, "mft_malloc: null out pointer");
    return g_alloc.alloc(bytes, as_stream(stream), ptr);
}
int32_t mft_free(void* ptr, mft_stream_t stream) { return g_alloc.release(ptr, as_stream(stream)); }
int32_t mft_empty_cache(void) {
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    g_alloc.release_cached_locked();
    return MFT_OK;
}
int32_t mft_trim_cache(int64_t keep_bytes) {
    MFT_CHECK_ARG(keep_bytes >= 0, "mft_trim_cache: negative size");
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    g_alloc.trim_locked(keep_bytes);
    return MFT_OK;
}
int32_t mft_mem_stats(int64_t* s) {
    MFT_CHECK_ARG(s != nullptr, "mft_mem_stats: null pointer");
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    s[0] = g_alloc.in_use; s[1] = g_alloc.cached; s[2] = g_alloc.peak; s[3] = g_alloc.n_cuda_malloc;
    s[4] = g_alloc.n_reuse; s[5] = g_alloc.n_cross_stream_waits;
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
