// Measurement aid: how many bytes per clock one SM takes in from L2 through its TMA unit when nothing else uses its
// shared memory.  One CTA per SM; one thread issues loads of an L2-resident bf16 matrix into a ring of 32 KB stages, a
// second thread waits for a stage and releases it at once.  No MMAs, no stores.  The tcgen05 GEMMs of this library
// are bound by operand delivery into shared memory; this kernel gives the ceiling of the delivery itself, for tensor
// boxes with 128-byte rows (what the GEMMs load) and for plain bulk copies of the same bytes.
#include <cuda.h>

#include <vector>

#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {
namespace {

using namespace ptx;

constexpr int PROBE_MAX_STAGES = 6, PROBE_STAGE_BYTES = 32768, PROBE_ROWS = 16384, PROBE_COLS = 2048;   // 64 MiB of bf16

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// mode 0: two tensor boxes of 128 rows x 128 bytes per stage; mode 1: two bulk copies of 16 KB; mode 2: one of each
__global__ void __launch_bounds__(64, 1)
tma_delivery_probe_kernel(const __grid_constant__ CUtensorMap map, const uint8_t* base, int mode, int stages, int iters, long long* cycles_out, int32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + PROBE_MAX_STAGES * PROBE_STAGE_BYTES);
    uint64_t* empty = full + PROBE_MAX_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + PROBE_MAX_STAGES);
    if (threadIdx.x == 0) {
        for (int s = 0; s < PROBE_MAX_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const long long t0 = clock64();
    constexpr int row_tiles = PROBE_ROWS / 128, kblocks = PROBE_COLS / 64;
    if (threadIdx.x == 0) {
        int stage = 0; uint32_t phase = 0;
        for (int it = 0; it < iters; ++it) {
            // a GEMM-like walk: two row tiles, the k-blocks of a row in order
            const int rt_a = (blockIdx.x * 2 + (it / kblocks) * 7) % row_tiles, rt_b = (rt_a + 1 + blockIdx.x) % row_tiles;
            const int kb = it % kblocks;
            if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;       // bounded
            mbar_arrive_expect_tx(&full[stage], PROBE_STAGE_BYTES);
            uint8_t* dst = tiles + stage * PROBE_STAGE_BYTES;
            if (mode == 0 || mode == 2) tma_load_2d(dst, &map, &full[stage], kb * 64, rt_a * 128);
            else bulk_load_1d(dst, base + ((size_t)rt_a * kblocks + kb) * 16384, 16384, &full[stage]);
            if (mode == 0) tma_load_2d(dst + 16384, &map, &full[stage], kb * 64, rt_b * 128);
            else bulk_load_1d(dst + 16384, base + ((size_t)rt_b * kblocks + kb) * 16384, 16384, &full[stage]);
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
    } else if (threadIdx.x == 32) {
        int stage = 0; uint32_t phase = 0;
        for (int it = 0; it < iters; ++it) {
            if (!mbar_wait(&full[stage], phase, abort_flag)) break;
            mbar_arrive(&empty[stage]);
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        cycles_out[blockIdx.x] = clock64() - t0;
        if (*abort_flag && status) atomicExch(status, MFT_ERR_TIMEOUT);
    }
}

}  // namespace
}  // namespace mft

using namespace mft;

extern "C" int32_t mft_probe_tma_delivery(int32_t mode, int32_t stages, int32_t ctas, int32_t iters, double* bytes_per_clock_per_sm_host,
                                          double* tb_per_s_host, mft_stream_t stream) {
    MFT_CHECK_ARG(mode >= 0 && mode <= 2 && stages >= 1 && stages <= PROBE_MAX_STAGES && ctas >= 1 && ctas <= 1024 && iters >= 1 && iters <= (1 << 20),
                  "mft_probe_tma_delivery: bad argument");
    MFT_CHECK_ARG(bytes_per_clock_per_sm_host && tb_per_s_host, "mft_probe_tma_delivery: null result pointer");
    if (!device_status_word()) return fail(MFT_ERR_INVALID_ARG, "mft_probe_tma_delivery: call mft_init first");
    cudaStream_t st = as_stream(stream);
    const size_t bytes = (size_t)PROBE_ROWS * PROBE_COLS * 2;
    void* buf = nullptr;
    long long* cycles = nullptr;
    if (int32_t s = check_cuda(cudaMalloc(&buf, bytes), "probe buffer")) return s;
    if (int32_t s = check_cuda(cudaMalloc(&cycles, sizeof(long long) * (size_t)ctas), "probe cycles")) { cudaFree(buf); return s; }
    int32_t rc = MFT_OK;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    do {
        if ((rc = check_cuda(cudaMemsetAsync(buf, 1, bytes, st), "probe memset"))) break;
        CUtensorMap map;
        if ((rc = make_tmap_bf16(&map, buf, PROBE_ROWS, PROBE_COLS, PROBE_COLS, 128))) break;
        const int smem = PROBE_MAX_STAGES * PROBE_STAGE_BYTES + 1024 + 256;
        static PerDeviceFlag configured_on;
        bool& configured = configured_on.here();
        if (!configured) {
            if ((rc = check_cuda(cudaFuncSetAttribute(tma_delivery_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "probe smem attr"))) break;
            configured = true;
        }
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        float ms = 0.f;
        for (int rep = 0; rep < 2; ++rep) {          // the first pass brings the matrix into L2
            cudaEventRecord(e0, st);
            tma_delivery_probe_kernel<<<ctas, 64, smem, st>>>(map, static_cast<const uint8_t*>(buf), mode, stages, iters, cycles, device_status_word());
            cudaEventRecord(e1, st);
            count_launch();
            if ((rc = check_cuda(cudaGetLastError(), "tma_delivery_probe"))) break;
            if ((rc = check_cuda(cudaEventSynchronize(e1), "probe sync"))) break;
            cudaEventElapsedTime(&ms, e0, e1);
        }
        if (rc) break;
        std::vector<long long> h((size_t)ctas);
        if ((rc = check_cuda(cudaMemcpy(h.data(), cycles, sizeof(long long) * (size_t)ctas, cudaMemcpyDeviceToHost), "probe read-back"))) break;
        long long longest = 1;
        for (long long v : h) longest = v > longest ? v : longest;
        *bytes_per_clock_per_sm_host = (double)iters * PROBE_STAGE_BYTES / (double)longest;
        *tb_per_s_host = (double)ctas * iters * PROBE_STAGE_BYTES / ((double)ms * 1e-3) / 1e12;
    } while (false);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(cycles);
    cudaFree(buf);
    return rc;
}
