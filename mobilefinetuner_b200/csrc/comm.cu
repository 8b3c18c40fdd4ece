// Data-parallel exchange of libmft_cuda.so: one communicator per process (one process per GPU), the sum of the
// flat f32 LoRA-gradient bucket after backward, and the status calls a host needs to notice a peer that is gone.
// The reference has no multi-device path; this is the only step of the sharded job where ranks exchange data.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that the kernel library loads on hosts without it and
// shares the copy a host program has already loaded.  Only the C API of nccl.h is used.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace {

using namespace mft;

struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclGetVersion) GetVersion = nullptr;
};

std::mutex g_mu;
NcclApi g_api;
ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 1;
bool g_aborted = false;

int32_t load_api() {
    if (g_api.handle) return MFT_OK;
    const char* names[] = {std::getenv("MFT_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(MFT_ERR_NCCL, "mft_comm: libnccl.so.2 not found (set MFT_NCCL_LIB to its path)");
    NcclApi a;
    a.handle = h;
#define BIND(field, sym)                                                          \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, sym));                 \
    if (!a.field) { dlclose(h); return fail(MFT_ERR_NCCL, std::string("mft_comm: NCCL lacks ") + sym); }
    BIND(GetUniqueId, "ncclGetUniqueId")
    BIND(CommInitRank, "ncclCommInitRank")
    BIND(AllReduce, "ncclAllReduce")
    BIND(CommAbort, "ncclCommAbort")
    BIND(CommDestroy, "ncclCommDestroy")
    BIND(CommGetAsyncError, "ncclCommGetAsyncError")
    BIND(GetErrorString, "ncclGetErrorString")
    BIND(GetVersion, "ncclGetVersion")
#undef BIND
    g_api = a;
    return MFT_OK;
}

int32_t check_nccl(ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return MFT_OK;
    return fail(MFT_ERR_NCCL, std::string(what) + ": " + (g_api.GetErrorString ? g_api.GetErrorString(r) : "NCCL error"));
}

int32_t usable(const char* who) {
    if (g_aborted) return fail(MFT_ERR_NCCL, std::string(who) + ": the communicator was aborted");
    if (!g_comm && g_world > 1) return fail(MFT_ERR_NCCL, std::string(who) + ": mft_comm_init has not been called");
    return MFT_OK;
}

template <typename T>
int32_t all_reduce(T* buf, int64_t n, ncclDataType_t dt, mft_stream_t stream, const char* who) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (int32_t s = usable(who)) return s;
    if (n < 0 || (n > 0 && !buf)) return fail(MFT_ERR_INVALID_ARG, std::string(who) + ": bad buffer");
    if (g_world == 1 || n == 0) return MFT_OK;
    return check_nccl(g_api.AllReduce(buf, buf, (size_t)n, dt, ncclSum, g_comm, as_stream(stream)), who);
}

}  // namespace

extern "C" {

int32_t mft_comm_unique_id(uint8_t* id_host) {
    MFT_CHECK_ARG(id_host, "mft_comm_unique_id: null buffer");
    std::lock_guard<std::mutex> lk(g_mu);
    if (int32_t s = load_api()) return s;
    static_assert(sizeof(ncclUniqueId) == MFT_COMM_ID_BYTES, "unique id size");
    ncclUniqueId id;
    if (int32_t s = check_nccl(g_api.GetUniqueId(&id), "ncclGetUniqueId")) return s;
    std::memcpy(id_host, &id, sizeof id);
    return MFT_OK;
}

int32_t mft_comm_init(int32_t rank, int32_t world, const uint8_t* id_host) {
    MFT_CHECK_ARG(world >= 1 && rank >= 0 && rank < world, "mft_comm_init: bad rank / world size");
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_comm) return fail(MFT_ERR_INVALID_ARG, "mft_comm_init: a communicator already exists (mft_comm_destroy first)");
    g_rank = rank; g_world = world; g_aborted = false;
    if (world == 1) return MFT_OK;                   // a single rank exchanges nothing: every call below is a no-op
    MFT_CHECK_ARG(id_host, "mft_comm_init: null unique id");
    if (int32_t s = load_api()) return s;
    ncclUniqueId id;
    std::memcpy(&id, id_host, sizeof id);
    ncclComm_t c = nullptr;
    if (int32_t s = check_nccl(g_api.CommInitRank(&c, world, id, rank), "ncclCommInitRank")) return s;
    g_comm = c;
    return MFT_OK;
}

int32_t mft_comm_info(int32_t* rank, int32_t* world, int32_t* nccl_version) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (rank) *rank = g_rank;
    if (world) *world = g_world;
    if (nccl_version) {
        int v = 0;
        if (g_api.GetVersion) g_api.GetVersion(&v);
        *nccl_version = v;
    }
    return MFT_OK;
}

int32_t mft_allreduce_sum_f32(float* buf, int64_t n, mft_stream_t stream) {
    return all_reduce(buf, n, ncclFloat32, stream, "mft_allreduce_sum_f32");
}

int32_t mft_allreduce_sum_i64(int64_t* buf, int64_t n, mft_stream_t stream) {
    return all_reduce(buf, n, ncclInt64, stream, "mft_allreduce_sum_i64");
}

int32_t mft_comm_async_error(int32_t* nccl_result_host) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (nccl_result_host) *nccl_result_host = 0;
    if (g_aborted) return fail(MFT_ERR_NCCL, "mft_comm_async_error: the communicator was aborted");
    if (!g_comm) return MFT_OK;
    ncclResult_t async = ncclSuccess;
    if (int32_t s = check_nccl(g_api.CommGetAsyncError(g_comm, &async), "ncclCommGetAsyncError")) return s;
    if (nccl_result_host) *nccl_result_host = (int32_t)async;
    if (async != ncclSuccess && async != ncclInProgress) return check_nccl(async, "asynchronous NCCL error");
    return MFT_OK;
}

int32_t mft_comm_wait(mft_stream_t stream, int32_t timeout_ms) {
    MFT_CHECK_ARG(timeout_ms > 0, "mft_comm_wait: the deadline must be positive");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaStreamQuery(as_stream(stream));
        if (q == cudaSuccess) return MFT_OK;
        if (q != cudaErrorNotReady) return check_cuda(q, "mft_comm_wait");
        cudaGetLastError();
        int32_t async = 0;
        if (int32_t s = mft_comm_async_error(&async)) { mft_comm_abort(); return s; }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > timeout_ms) {
            mft_comm_abort();
            return fail(MFT_ERR_TIMEOUT, "mft_comm_wait: the exchange did not finish before the deadline; communicator aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

int32_t mft_comm_abort(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_comm) {
        g_api.CommAbort(g_comm);
        g_comm = nullptr;
    }
    g_aborted = g_world > 1;
    return MFT_OK;
}

int32_t mft_comm_destroy(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    int32_t s = MFT_OK;
    if (g_comm) {
        s = check_nccl(g_api.CommDestroy(g_comm), "ncclCommDestroy");
        g_comm = nullptr;
    }
    g_rank = 0; g_world = 1; g_aborted = false;
    return s;
}

}  // extern "C"
