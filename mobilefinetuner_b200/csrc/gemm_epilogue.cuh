// Shared epilogue of the tcgen05 GEMM kernels for bf16 outputs: one warp moves its 32 accumulator rows of a
// tile from tensor memory through registers into swizzled shared-memory boxes (32 rows x 64 columns) and
// stores them with TMA tensor stores (coalesced 128-byte rows; rows / columns outside D are clipped by the
// tensor map).  The element-wise part depends on the mode:
//   EPI_STORE   : alpha * acc + bias
//   EPI_CE_GRAD : (exp(acc - lse[row]) - [col == label[row]]) * dloss / n_valid
//   EPI_CE_P    : exp(acc - m_ref[row]) (un-normalised softmax numerators), plus the per-row sum of the values
//                 stored, the label logit, and a per-row flag when acc - m_ref is too large to trust
#pragma once
#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

constexpr int EPI_BOX_BYTES = 32 * 64 * 2;
// EPI_CE_P trusts exp(acc - m_ref) only up to e^60 (the row sum over a 2^18-entry vocabulary stays finite in fp32);
// rows beyond it are flagged and recomputed exactly by the caller.
constexpr float CE_P_MAX_EXCESS = 60.f;

template <int EPI, int BN>
__device__ __forceinline__ void epilogue_bf16_tma(const GemmParams& p, const CUtensorMap* map_d, uint8_t* store_smem, uint32_t taddr,
                                                  int q, int lane, int row, int store_row0, int n0, int& box_ctr) {
    using namespace ptx;
    float lse = 0.f, coef = 0.f, row_sum = 0.f;
    int tgt = -1;
    if constexpr (EPI == EPI_CE_GRAD || EPI == EPI_CE_P) {
        if (row < p.m) {
            tgt = p.ce_tgt[row];
            lse = p.ce_lse[row];                 // EPI_CE_P: the reference value m_ref[row]
            if constexpr (EPI == EPI_CE_GRAD) {
                const long long nv = p.ce_nvalid_override > 0 ? p.ce_nvalid_override : (long long)*p.ce_nvalid;
                coef = (tgt >= 0 && nv > 0) ? p.ce_dloss / (float)nv : 0.f;
            }
            tgt -= p.ce_col_offset;
        }
    }
#pragma unroll 1
    for (int c = 0; c < BN; c += 64) {
        if (n0 + c >= p.n) break;          // uniform across the warp
        uint8_t* buf = store_smem + (q * 2 + (box_ctr & 1)) * EPI_BOX_BYTES;
        const uint32_t buf_addr = smem_u32(buf) + (uint32_t)lane * 128u;
        if (lane == 0) tma_store_wait_read<1>();   // the store that last used this buffer has read it
        __syncwarp();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + (uint32_t)(c + half * 32), r);
            tmem_ld_wait();
            const int col0 = n0 + c + half * 32;
            float v[32];
            if constexpr (EPI == EPI_STORE) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) if (col0 + j < p.n) v[j] += __ldg(p.bias + col0 + j);
                }
            } else if constexpr (EPI == EPI_CE_GRAD) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float pr = __expf(__uint_as_float(r[j]) * p.alpha - lse);
                    v[j] = (pr - (col0 + j == tgt ? 1.f : 0.f)) * coef;
                }
            } else {
                float dmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float l = __uint_as_float(r[j]) * p.alpha;
                    if (col0 + j == tgt && row < p.m) p.ce_tgt_logit[row] = l;
                    const float d = (col0 + j < p.n) ? l - lse : -INFINITY;
                    dmax = fmaxf(dmax, d);
                    v[j] = __bfloat162float(__float2bfloat16_rn(__expf(d)));     // the value GEMM 2 will see
                    row_sum += v[j];
                }
                if (dmax > CE_P_MAX_EXCESS && row < p.m) p.ce_flag[row] = 1;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pos = (uint32_t)((half * 4 + j) ^ (lane & 7));   // 128-byte swizzle
                const __nv_bfloat162 w0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
                const __nv_bfloat162 w1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                const __nv_bfloat162 w2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                const __nv_bfloat162 w3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                st_shared_v4(buf_addr + pos * 16u, *reinterpret_cast<const uint32_t*>(&w0), *reinterpret_cast<const uint32_t*>(&w1),
                             *reinterpret_cast<const uint32_t*>(&w2), *reinterpret_cast<const uint32_t*>(&w3));
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_d, buf, n0 + c, store_row0);
            tma_store_commit();
        }
        ++box_ctr;
    }
    if constexpr (EPI == EPI_CE_P) {
        if (row < p.m) p.ce_partials[(long long)row * p.ce_partial_ld + (p.ce_col_offset + n0) / CE_TILE_N] = make_float2(0.f, row_sum);
    }
}

// f32 outputs: boxes of 32 rows x 32 columns (128-byte rows, same swizzle), written with a tensor store or,
// when D already holds a partial result (accumulate / K split), added to memory by a tensor reduction.
template <int BN>
__device__ __forceinline__ void epilogue_f32_tma(const GemmParams& p, const CUtensorMap* map_d, uint8_t* store_smem, uint32_t taddr,
                                                 int q, int lane, int store_row0, int n0, bool add_bias, int& box_ctr) {
    using namespace ptx;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.n) break;          // uniform across the warp
        uint8_t* buf = store_smem + (q * 2 + (box_ctr & 1)) * EPI_BOX_BYTES;
        const uint32_t buf_addr = smem_u32(buf) + (uint32_t)lane * 128u;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint32_t r[32];
        tmem_ld_32x32(taddr + (uint32_t)c, r);
        tmem_ld_wait();
        const int col0 = n0 + c;
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * p.alpha);
        if (add_bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < p.n) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(p.bias + col0 + j));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t pos = (uint32_t)(j ^ (lane & 7));   // 128-byte swizzle
            st_shared_v4(buf_addr + pos * 16u, r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            if (p.f32_reduce) tma_reduce_add_2d(map_d, buf, col0, store_row0);
            else tma_store_2d(map_d, buf, col0, store_row0);
            tma_store_commit();
        }
        ++box_ctr;
    }
}

}  // namespace mft
