// "TN" GEMM with the long token dimension contracted:
//     out[p,q] += alpha * sum_t U[t,p] * V[t,q]        (U [T,P], V [T,Q] bf16 row-major)
// This is the shape of the LoRA weight gradients (dA = X^T (dY B^T), dB = (XA)^T dY):
// one of P,Q is the padded rank panel (64), T is 10^3..10^5.  The kernel is bound
// by reading U and V once from HBM; the tiny fp32 result is reduced across the
// T-splits with atomics.  Warp-level mma.sync (m16n8k16, bf16 -> f32) with
// ldmatrix.trans on both operands, cp.async double buffering.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

constexpr int TN_PT = 128;      // p-tile
constexpr int TN_QT = 64;       // q-tile
constexpr int TN_TC = 64;       // tokens per pipeline step
constexpr int TN_STAGES = 3;    // cp.async ring depth
constexpr int TN_THREADS = 256;
constexpr int TN_US = TN_PT + 8;   // padded row strides (elements): conflict-free ldmatrix
constexpr int TN_VS = TN_QT + 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int sz = valid ? 16 : 0;   // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(TN_THREADS)
gemm_tn_kernel(const __nv_bfloat16* __restrict__ U, int64_t ldu, const __nv_bfloat16* __restrict__ V, int64_t ldv,
               int64_t T, int P, int Q, float alpha, float* __restrict__ out, int64_t stride_p, int64_t stride_q, int64_t t_per_split) {
    dep_trigger();
    dep_wait();
    extern __shared__ __align__(16) uint8_t tn_smem[];
    typedef __nv_bfloat16 (*UsT)[TN_TC][TN_US];
    typedef __nv_bfloat16 (*VsT)[TN_TC][TN_VS];
    UsT Us = reinterpret_cast<UsT>(tn_smem);
    VsT Vs = reinterpret_cast<VsT>(tn_smem + sizeof(__nv_bfloat16) * TN_STAGES * TN_TC * TN_US);
    const int p0 = blockIdx.x * TN_PT, q0 = blockIdx.y * TN_QT;
    const int64_t t_begin = (int64_t)blockIdx.z * t_per_split;
    const int64_t t_end = min(T, t_begin + t_per_split);
    if (t_begin >= t_end) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsteps = (int)((t_end - t_begin + TN_TC - 1) / TN_TC);
    // 8-column blocks of the q-tile that exist (in pairs): a rank-16 panel costs a quarter of the MMAs of a full tile
    const int nb_lim = min(8, ((Q - q0 + 15) / 16) * 2);

    auto load_step = [&](int step, int buf) {
        const int64_t t0 = t_begin + (int64_t)step * TN_TC;
        // U chunk: 32 rows x 16 vectors of 8
        for (int i = threadIdx.x; i < TN_TC * (TN_PT / 8); i += TN_THREADS) {
            const int r = i / (TN_PT / 8), c = (i % (TN_PT / 8)) * 8;
            const bool ok = (t0 + r < t_end) && (p0 + c < P);
            cp_async16(&Us[buf][r][c], ok ? U + (t0 + r) * ldu + p0 + c : U, ok);
        }
        for (int i = threadIdx.x; i < TN_TC * (TN_QT / 8); i += TN_THREADS) {
            const int r = i / (TN_QT / 8), c = (i % (TN_QT / 8)) * 8;
            const bool ok = (t0 + r < t_end) && (q0 + c < Q);
            cp_async16(&Vs[buf][r][c], ok ? V + (t0 + r) * ldv + q0 + c : V, ok);
        }
        cp_async_commit();
    };

    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // prologue: fill STAGES-1 slots (empty commit groups keep the group count uniform)
    for (int s = 0; s < TN_STAGES - 1; ++s) {
        if (s < nsteps) load_step(s, s); else cp_async_commit();
    }
    for (int step = 0; step < nsteps; ++step) {
        const int buf = step % TN_STAGES;
        cp_async_wait<TN_STAGES - 2>();      // the group of `step` has landed
        __syncthreads();                     // ...for every thread, and slot (step-1)%STAGES is free again
        if (step + TN_STAGES - 1 < nsteps) load_step(step + TN_STAGES - 1, (step + TN_STAGES - 1) % TN_STAGES);
        else cp_async_commit();
#pragma unroll
        for (int kk = 0; kk < TN_TC; kk += 16) {
            uint32_t a[4];
            {   // A = U^T tile: rows p (16 per warp), cols t
                const int t = kk + (lane & 7) + ((lane >> 4) << 3);
                const int p = warp * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(a, &Us[buf][t][p]);
            }
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                if (nb >= nb_lim) break;
                uint32_t b[4];
                const int t = kk + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int q = nb * 8 + (lane >> 4) * 8;
                ldmatrix_x4_trans(b, &Vs[buf][t][q]);
                mma_bf16_16816(acc[nb], a, b[0], b[1]);
                mma_bf16_16816(acc[nb + 1], a, b[2], b[3]);
            }
        }
    }
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = p0 + warp * 16 + g + h * 8;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int q = q0 + nb * 8 + tq * 2 + e;
                if (p < P && q < Q) atomicAdd(out + (int64_t)p * stride_p + (int64_t)q * stride_q, alpha * acc[nb][h * 2 + e]);
            }
        }
    }
}


// ---------------------------------------------------------------- the same product on the tensor-memory path
// U^T V with the token dimension as the MMA's K: both operands are consumed exactly as they lie in memory (rows =
// tokens, features contiguous), i.e. as "MN-major" A and B operands of tcgen05.mma; nothing is transposed.
// One CTA per (128 U-columns, 64 V-columns, token range): warp 0 streams [64 tokens x 64 columns] boxes with TMA
// (128-byte swizzle, 4 stages), warp 1's one thread issues 4 MMAs per 64 tokens into a 128 x 64 f32 accumulator in
// tensor memory, warps 2..5 add the result into `out` with f32 atomics (the token ranges of a tile meet there).
namespace tn_tc {
using namespace ptx;
constexpr int PT = 128, QT = 64, TC = 64, STAGES = 4, THREADS = 192;
constexpr int U_BYTES = 2 * TC * 128, V_BYTES = TC * 128, STAGE_BYTES = U_BYTES + V_BYTES;     // 16 KB + 8 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;

__device__ __forceinline__ uint64_t desc_mn(uint32_t addr, uint32_t chunk_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((chunk_bytes >> 4) & 0x3FFF) << 16;     // distance between 64-column chunks
    d |= (uint64_t)(1024 >> 4) << 32;                       // 8 token rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(THREADS)
gemm_tn_tc_kernel(const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_v, int64_t T, int P, int Q,
                  float alpha, float* __restrict__ out, int64_t stride_p, int64_t stride_q, int64_t t_per_split, int32_t* status) {
    dep_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* full_bar = bars;              // [STAGES]
    uint64_t* empty_bar = bars + STAGES;    // [STAGES]
    uint64_t* done_bar = bars + 2 * STAGES; // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * PT, q0 = blockIdx.y * QT;
    const int64_t t_begin = (int64_t)blockIdx.z * t_per_split;
    const int64_t t_end = min(T, t_begin + t_per_split);
    const int nsteps = t_begin < t_end ? (int)((t_end - t_begin + TC - 1) / TC) : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(done_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_u); tma_prefetch_desc(&map_v);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    dep_wait();
    if (nsteps > 0) {
        if (warp == 0) {
            if (lane == 0) {
                for (int s = 0; s < nsteps; ++s) {
                    const int st = s % STAGES;
                    const uint32_t ph = (s / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[st], ph ^ 1, abort_flag)) break;
                    uint8_t* u = tiles + st * STAGE_BYTES;
                    const int row = (int)(t_begin + (int64_t)s * TC);
                    mbar_arrive_expect_tx(&full_bar[st], STAGE_BYTES);
                    tma_load_2d(u, &map_u, &full_bar[st], p0, row);
                    tma_load_2d(u + TC * 128, &map_u, &full_bar[st], p0 + 64, row);
                    tma_load_2d(u + U_BYTES, &map_v, &full_bar[st], q0, row);
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                const int n_eff = min(QT, (Q - q0 + 15) & ~15);
                const uint32_t idesc = idesc_bf16_f32(PT, (uint32_t)n_eff) | (1u << 15) | (1u << 16);    // A and B MN-major
                bool ok = true;
                for (int s = 0; s < nsteps && ok; ++s) {
                    const int st = s % STAGES;
                    const uint32_t ph = (s / STAGES) & 1;
                    if (!mbar_wait(&full_bar[st], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t ua = smem_u32(tiles + st * STAGE_BYTES);
                    const uint64_t ud = desc_mn(ua, TC * 128), vd = desc_mn(ua + U_BYTES, TC * 128);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_bf16(tmem_base, ud + (uint64_t)(j * (2048 / 16)), vd + (uint64_t)(j * (2048 / 16)), idesc, (s | j) != 0 ? 1u : 0u);
                    umma_commit(&empty_bar[st]);
                }
                if (ok) umma_commit(done_bar);
            }
        } else {
            const int q4 = warp & 3;
            const int p = p0 + q4 * 32 + lane;
            if (mbar_wait(done_bar, 0, abort_flag)) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < QT; c += 32) {
                    if (q0 + c >= Q) break;
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c, r);
                    tmem_ld_wait();
                    if (p < P) {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (q0 + c + x < Q) atomicAdd(out + (int64_t)p * stride_p + (int64_t)(q0 + c + x) * stride_q, alpha * __uint_as_float(r[x]));
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, MFT_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 64);
    }
}
}  // namespace tn_tc

}  // namespace mft

using namespace mft;

extern "C" int32_t mft_gemm_tn_acc(const void* u, int64_t ldu, const void* v, int64_t ldv, int64_t t, int64_t p, int64_t q,
                                   float alpha, float* out, int64_t ldo, mft_stream_t stream) {
    MFT_CHECK_ARG(u && v && out && t > 0 && p > 0 && q > 0, "mft_gemm_tn_acc: bad argument");
    MFT_CHECK_ARG(p % 8 == 0 && q % 8 == 0 && ldu % 8 == 0 && ldv % 8 == 0, "mft_gemm_tn_acc: P, Q and the row strides must be multiples of 8");
    MFT_CHECK_ARG(reinterpret_cast<uintptr_t>(u) % 16 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0, "mft_gemm_tn_acc: operands must be 16-byte aligned");
    MFT_CHECK_ARG(ldo >= q && p < (1 << 30) && q < (1 << 30), "mft_gemm_tn_acc: bad leading dimension");
    // The kernel streams a 128-column slab of U and a 64-column slab of V: put the wide operand on the U side
    // (longer contiguous row pieces) and write the result transposed when the operands are swapped.
    const bool swap = q > p;
    const void* uu = swap ? v : u; const void* vv = swap ? u : v;
    const int64_t ldu2 = swap ? ldv : ldu, ldv2 = swap ? ldu : ldv;
    const int64_t pp = swap ? q : p, qq = swap ? p : q;
    const int64_t stride_p = swap ? 1 : ldo, stride_q = swap ? ldo : 1;
    const int tiles_p = (int)((pp + TN_PT - 1) / TN_PT), tiles_q = (int)((qq + TN_QT - 1) / TN_QT);
    const int64_t tiles = (int64_t)tiles_p * tiles_q;
    // Split T so that the CTAs fill whole waves (2 resident CTAs per SM): per wave a CTA streams its token range
    // plus a fixed pipeline-fill / atomic-flush part worth ~256 tokens.
    const int64_t slots = 148 * 2;
    const int64_t max_splits = std::min<int64_t>(65535, std::max<int64_t>(1, (t + 2 * TN_TC - 1) / (2 * TN_TC)));
    int64_t splits = 1;
    double best = 1e300;
    for (int64_t sp = 1; sp <= max_splits && sp <= 4096; ++sp) {
        const int64_t per = ((t + sp - 1) / sp + TN_TC - 1) / TN_TC * TN_TC;
        const int64_t waves = (tiles * sp + slots - 1) / slots;
        const double cost = (double)waves * (double)(per + 256);
        if (cost < best) { best = cost; splits = sp; }
    }
    int64_t t_per = (t + splits - 1) / splits;
    t_per = (t_per + TN_TC - 1) / TN_TC * TN_TC;
    splits = (t + t_per - 1) / t_per;
    MFT_CHECK_ARG(tiles_q <= 65535, "mft_gemm_tn_acc: Q too large");
    // Tensor-memory kernel: same tiles, 2 resident CTAs per SM.  Measured at 16384 tokens, rank 16: 42.5 us against
    // 56.5 us at P = 6912 (5.3 TB/s), but 15.4 against 13.9 us at P = 1152, where each CTA streams only 8 boxes and its
    // set-up (barriers, tensor-memory allocation) shows; so it takes the wide products only.
    // MFT_TN_TC=0 keeps the mma.sync kernel everywhere, MFT_TN_TC=2 uses this one wherever it applies.
    static const int use_tc = [] { const char* e = std::getenv("MFT_TN_TC"); return e ? std::atoi(e) : 1; }();
    if (use_tc && device_status_word() && pp >= (use_tc >= 2 ? 64 : 2048) && t < (1ll << 31)) {
        // token ranges in whole 64-token boxes, so that no box straddles two ranges
        t_per = (t_per + tn_tc::TC - 1) / tn_tc::TC * tn_tc::TC;
        splits = (t + t_per - 1) / t_per;
        CUtensorMap mu, mv;
        if (make_tmap_bf16(&mu, uu, t, pp, ldu2, tn_tc::TC) == MFT_OK && make_tmap_bf16(&mv, vv, t, qq, ldv2, tn_tc::TC) == MFT_OK) {
            static PerDeviceFlag tc_configured_on;           // function attributes are per device
            bool& tc_configured = tc_configured_on.here();
            if (!tc_configured) {
                if (int32_t s = check_cuda(cudaFuncSetAttribute(tn_tc::gemm_tn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tn_tc::SMEM_BYTES), "gemm_tn smem attr")) return s;
                tc_configured = true;
            }
            dim3 grid_tc((unsigned)tiles_p, (unsigned)tiles_q, (unsigned)splits);
            launch_dep(tn_tc::gemm_tn_tc_kernel, grid_tc, dim3(tn_tc::THREADS), (size_t)tn_tc::SMEM_BYTES, as_stream(stream), mu, mv, t, (int)pp, (int)qq,
                       alpha, out, stride_p, stride_q, t_per, device_status_word());
            MFT_LAUNCH_CHECK("gemm_tn_tc");
            return MFT_OK;
        }
    }
    dim3 grid((unsigned)tiles_p, (unsigned)tiles_q, (unsigned)splits);
    constexpr int smem = (int)(sizeof(__nv_bfloat16) * TN_STAGES * TN_TC * (TN_US + TN_VS));
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gemm_tn smem attr")) return s;
        configured = true;
    }
    launch_dep(gemm_tn_kernel, dim3(grid), dim3(TN_THREADS), (size_t)(smem), as_stream(stream), (const __nv_bfloat16*)uu, ldu2, (const __nv_bfloat16*)vv, ldv2, t,
                                                                  (int)pp, (int)qq, alpha, out, stride_p, stride_q, t_per);
    MFT_LAUNCH_CHECK("gemm_tn");
    return MFT_OK;
}
