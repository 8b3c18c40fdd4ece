// Shared epilogue of the tcgen05 GEMM kernels for bf16 outputs: one warp moves its 32 accumulator rows of a
// tile from tensor memory through registers into swizzled shared-memory boxes (32 rows x 64 columns) and
// stores them with TMA tensor stores (coalesced 128-byte rows; rows / columns outside D are clipped by the
// tensor map).  The element-wise part depends on the mode:
//   EPI_STORE   : alpha * acc + bias
//   EPI_CE_GRAD : (exp(acc - lse[row]) - [col == label[row]]) * dloss / n_valid
//   EPI_CE_P    : exp(acc - m_ref[row]) (un-normalised softmax numerators), plus the per-row sum of the values
//                 stored, the label logit, and a per-row flag when acc - m_ref is too large to trust
#pragma once
#include "act_math.cuh"
#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

constexpr int EPI_BOX_BYTES = 32 * 64 * 2;

// The CTA-pair kernel runs two epilogue warps per lane quadrant of tensor memory (a warp reaches only the 32 lanes
// warp % 4 selects).  They share the quadrant's boxes: each fills one half of a box's columns, the `owner` (side 0)
// waits until the previous store from the box has read it, tells the `helper` (side 1), and issues the TMA store once
// the helper's half is in.  The per-element work of an epilogue is what bounds it (one warp per scheduler cannot hide
// the latency of its own tensor-memory loads and special-function chains), so two warps per quadrant nearly halve it.
// side -1: one warp fills the whole box (single-CTA kernel).  All waits are bounded.
struct BoxPair {
    uint64_t* free_bar = nullptr;     // owner -> helper: the box may be written            (count 1, one phase per box);
                                      // gated-MLP backward: the owner has taken the helper's report of a chunk
    uint64_t* filled_bar = nullptr;   // helper -> owner: the helper's half is in the box   (count 1, one phase per box)
    uint64_t* sum_bar = nullptr;      // helper -> owner: per-row sums of a tile are in `sums` (EPI_CE_P; one phase per tile)
    float* sums = nullptr;            // [32] floats of this quadrant
    volatile int* abort_flag = nullptr;
    int side = -1;
    int uses = 0, tiles = 0;
    __device__ __forceinline__ int half_begin() const { return side == 1 ? 1 : 0; }
    __device__ __forceinline__ int half_end() const { return side == 0 ? 1 : 2; }
};
// Before a box is written.  PENDING = stores that may still be reading OTHER boxes of this warp.
template <int PENDING>
__device__ __forceinline__ bool box_acquire(BoxPair& bp, int lane) {
    using namespace ptx;
    if (bp.side == 1) return __all_sync(0xffffffffu, mbar_wait(bp.free_bar, (uint32_t)(bp.uses & 1), bp.abort_flag)) != 0;   // the same answer in every lane
    if (lane == 0) {
        tma_store_wait_read<PENDING>();
        if (bp.side == 0) mbar_arrive(bp.free_bar);
    }
    __syncwarp();
    return true;
}
// After a box is written.  Returns true in the warp whose lane 0 issues the store; `ok` turns false when a wait ran out.
__device__ __forceinline__ bool box_release(BoxPair& bp, int lane, bool& ok) {
    using namespace ptx;
    fence_proxy_async();
    __syncwarp();
    if (bp.side == 1) {
        if (lane == 0) mbar_arrive(bp.filled_bar);
        ++bp.uses;
        return false;
    }
    if (bp.side == 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bp.filled_bar, (uint32_t)(bp.uses & 1), bp.abort_flag)) != 0;
        ++bp.uses;
    }
    return ok;
}
// EPI_CE_P trusts exp(acc - m_ref) only up to e^60 (the row sum over a 2^18-entry vocabulary stays finite in fp32);
// rows beyond it are flagged and recomputed exactly by the caller.
constexpr float CE_P_MAX_EXCESS = 60.f;

template <int EPI, int BN>
__device__ __forceinline__ bool epilogue_bf16_tma(const GemmParams& p, const CUtensorMap* map_d, uint8_t* store_smem, uint32_t taddr,
                                                  int q, int lane, int row, int store_row0, int n0, int& box_ctr, BoxPair& bp) {
    using namespace ptx;
    bool ok = true;
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
        if (!box_acquire<1>(bp, lane)) return false;   // the store that last used this buffer has read it
        for (int half = bp.half_begin(); half < bp.half_end(); ++half) {
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
        if (box_release(bp, lane, ok) && lane == 0) {
            tma_store_2d(map_d, buf, n0 + c, store_row0);
            tma_store_commit();
        }
        if (!ok) return false;
        ++box_ctr;
    }
    if constexpr (EPI == EPI_CE_P) {
        if (bp.side == 1) {                  // the helper hands its part of the row sums to the owner
            bp.sums[lane] = row_sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(bp.sum_bar);
        } else {
            if (bp.side == 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(bp.sum_bar, (uint32_t)(bp.tiles & 1), bp.abort_flag))) return false;
                row_sum += bp.sums[lane];
            }
            if (row < p.m) p.ce_partials[(long long)row * p.ce_partial_ld + (p.ce_col_offset + n0) / CE_TILE_N] = make_float2(0.f, row_sum);
        }
        ++bp.tiles;
    }
    return true;
}

// ---- gated MLP, forward.  The accumulator of this CTA holds 128 rows x [128 gate columns | 128 up columns].  Per
// 64-column chunk the warp writes three boxes: the gate chunk and the up chunk into D (the saved gate|up activation,
// at their natural columns g0 + c and inter + g0 + c) and f(gate) * up into the act tensor.  Gate and up are rounded
// to bf16 before the gating, so the result is bit-identical to the stand-alone activation kernel on the stored values.
__device__ __forceinline__ void epi_pack_store_half(uint32_t buf_addr, int half, int lane, const float (&v)[32]) {
    using namespace ptx;
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
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ bool epilogue_glu_fwd(const GemmParams& p, const CUtensorMap* map_d, const CUtensorMap* map_act, uint8_t* store_smem,
                                                 uint32_t taddr, int q, int lane, int store_row0, int g0, int& box_ctr, BoxPair& bp) {
    using namespace ptx;
    const bool geglu = p.glu_geglu != 0;
    bool ok = true;
#pragma unroll 1
    for (int c = 0; c < 128; c += 64) {
        // pass 0: gate chunk -> D, pass 1: up chunk -> D, pass 2: f(gate) * up -> act
#pragma unroll 1
        for (int pass = 0; pass < 3; ++pass) {
            uint8_t* buf = store_smem + (q * 2 + (box_ctr & 1)) * EPI_BOX_BYTES;
            const uint32_t buf_addr = smem_u32(buf) + (uint32_t)lane * 128u;
            if (!box_acquire<1>(bp, lane)) return false;   // the store that last used this buffer has read it
            for (int half = bp.half_begin(); half < bp.half_end(); ++half) {
                float v[32];
                if (pass < 2) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)(pass * 128 + c + half * 32), r);
                    tmem_ld_wait();
                    const int col0 = pass * p.glu_inter + g0 + c + half * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += __ldg(p.bias + col0 + j);
                    }
                } else {
                    uint32_t rg[32], ru[32];
                    tmem_ld_32x32(taddr + (uint32_t)(c + half * 32), rg);
                    tmem_ld_32x32(taddr + (uint32_t)(128 + c + half * 32), ru);
                    tmem_ld_wait();
                    const int colg = g0 + c + half * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float g = __uint_as_float(rg[j]) * p.alpha, u = __uint_as_float(ru[j]) * p.alpha;
                        if (p.bias) { g += __ldg(p.bias + colg + j); u += __ldg(p.bias + p.glu_inter + colg + j); }
                        v[j] = glu_fwd(geglu, round_bf16(g), round_bf16(u));
                    }
                }
                epi_pack_store_half(buf_addr, half, lane, v);
            }
            if (box_release(bp, lane, ok) && lane == 0) {
                if (pass < 2) tma_store_2d(map_d, buf, pass * p.glu_inter + g0 + c, store_row0);
                else tma_store_2d(map_act, buf, g0 + c, store_row0);
                tma_store_commit();
            }
            if (!ok) return false;
            ++box_ctr;
        }
    }
    return true;
}

__device__ __forceinline__ uint32_t ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
    return a;
}

// ---- staged epilogue of the 256 x 384 tile (bf16 outputs).  The CTA's 128 x 384 accumulator goes, rounded to bf16, into
// 24 boxes of 32 rows x 64 columns (box = quadrant * 6 + 64-column chunk of the accumulator), the tensor memory is
// released, and the boxes are stored afterwards.  `side` 0 / 1 = the warp's 32-column half of every chunk.
// Gated MLP: the chunks of the accumulator are gate 0, gate 1, up 0, up 1, gate 2, up 2 (64 columns each).
__device__ __forceinline__ int staged_glu_kind(int chunk) { return (0x2C >> chunk) & 1; }           // 1 = up
__device__ __forceinline__ int staged_glu_index(int chunk) { return chunk < 4 ? (chunk & 1) : 2; }   // 64-column block within gate / up
// Chunks [CH0, CH1) of the accumulator.  The tensor-memory load of the next chunk is in flight while this one is
// scaled, rounded and written (tcgen05.wait::ld waits for every load issued before it, so the next load is issued
// after the wait and before the arithmetic).
template <int EPI, int CH0, int CH1>
__device__ __forceinline__ void staged_drain(const GemmParams& p, uint8_t* staging, uint32_t taddr, int q, int side, int lane, int n0) {
    using namespace ptx;
    uint32_t r[2][32];
    tmem_ld_32x32(taddr + (uint32_t)(CH0 * 64 + side * 32), r[0]);
    tmem_ld_wait();
#pragma unroll
    for (int ch = CH0; ch < CH1; ++ch) {
        const int cur = (ch - CH0) & 1;
        if (ch + 1 < CH1) tmem_ld_32x32(taddr + (uint32_t)((ch + 1) * 64 + side * 32), r[cur ^ 1]);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[cur][j]) * p.alpha;
        if (p.bias) {
            const int col0 = (EPI == EPI_GLU_FWD ? staged_glu_kind(ch) * p.glu_inter + n0 + staged_glu_index(ch) * 64 : n0 + ch * 64) + side * 32;
            const int col_end = EPI == EPI_GLU_FWD ? 2 * p.glu_inter : p.n;     // a ragged last tile of the plain store
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < col_end) v[j] += __ldg(p.bias + col0 + j);
        }
        epi_pack_store_half(smem_u32(staging + (q * 6 + ch) * EPI_BOX_BYTES) + (uint32_t)lane * 128u, side, lane, v);
        if (ch + 1 < CH1) tmem_ld_wait();
    }
}
// Plain store: epilogue warp `ew` of 8 stores boxes ew, ew + 8, ew + 16 (one lane issues).
__device__ __forceinline__ void staged_store_plain(const CUtensorMap* map_d, uint8_t* staging, int ew, int lane, int m0, int n0, int n) {
    using namespace ptx;
    if (lane != 0) return;
    for (int b = ew; b < 24; b += 8)
        if (n0 + (b % 6) * 64 < n)          // boxes past the last column of a ragged tile are not stored; a box across it is clipped
            tma_store_2d(map_d, staging + b * EPI_BOX_BYTES, n0 + (b % 6) * 64, m0 + (b / 6) * 32);
    tma_store_commit();
}
// Gated MLP: epilogue warp `ew` takes the (gate, up) box pairs ew and ew + 8 of the CTA's 12 (quadrant * 3 + block): it
// forms f(gate) * up of its 32 rows x 64 columns from the staged bf16 values (bit-identical to the stand-alone
// activation kernel on the stored tensors), stores the gate and up boxes into D, waits until those stores have read
// them, writes the result over the gate box and stores that into the act tensor.
__device__ __forceinline__ void staged_store_glu(const GemmParams& p, const CUtensorMap* map_d, const CUtensorMap* map_act, uint8_t* staging,
                                                 int ew, int lane, int m0, int g0) {
    using namespace ptx;
    const bool geglu = p.glu_geglu != 0;
#pragma unroll 1
    for (int pr = ew; pr < 12; pr += 8) {
        const int qq = pr / 3, j = pr % 3;
        uint8_t* gbox = staging + (qq * 6 + (j < 2 ? j : 4)) * EPI_BOX_BYTES;
        uint8_t* ubox = staging + (qq * 6 + (j < 2 ? 2 + j : 5)) * EPI_BOX_BYTES;
        const uint32_t g_addr = smem_u32(gbox) + (uint32_t)lane * 128u, u_addr = smem_u32(ubox) + (uint32_t)lane * 128u;
        uint32_t act[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t pos = (uint32_t)(u ^ (lane & 7)) * 16u;
            uint32_t gw[4], uw[4];
            ld_shared_v4(g_addr + pos, gw[0], gw[1], gw[2], gw[3]);
            ld_shared_v4(u_addr + pos, uw[0], uw[1], uw[2], uw[3]);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[w]));
                const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[w]));
                const __nv_bfloat162 a2 = __floats2bfloat162_rn(glu_fwd(geglu, g2.x, u2.x), glu_fwd(geglu, g2.y, u2.y));
                act[4 * u + w] = *reinterpret_cast<const uint32_t*>(&a2);
            }
        }
        __syncwarp();                           // every lane has read its rows of both boxes
        if (lane == 0) {
            tma_store_2d(map_d, gbox, g0 + j * 64, m0 + qq * 32);
            tma_store_2d(map_d, ubox, p.glu_inter + g0 + j * 64, m0 + qq * 32);
            tma_store_commit();
            tma_store_wait_read<0>();
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 8; ++u)
            st_shared_v4(g_addr + (uint32_t)(u ^ (lane & 7)) * 16u, act[4 * u], act[4 * u + 1], act[4 * u + 2], act[4 * u + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_act, gbox, g0 + j * 64, m0 + qq * 32);
            tma_store_commit();
        }
    }
}

// ---- gated MLP, backward.  The accumulator holds d(act) for 128 rows x 256 columns of [M, inter].  Per 64-column
// chunk the warp loads the matching boxes of the saved gate and up activations with TMA (GLU_SETS sets of two boxes per
// warp: the loads of the next chunk are in flight while this one is computed), forms d_gate and d_up IN PLACE in those
// boxes and stores them to D at columns n and inter + n.  d(act) is rounded to bf16 first, so the result is
// bit-identical to the stand-alone backward kernel fed with a stored bf16 d(act).
// (gate, up) box sets per warp: chunk k computes in set k % GLU_SETS while the loads of the following GLU_SETS - 1 chunks
// are in flight.  Measured at 16384 x 6912 x 1152: two sets with five pipeline stages 0.377 ms, three sets with four
// stages 0.388 ms (against 0.228 + 0.203 ms for the GEMM and the stand-alone kernel): the epilogue is bound by its own
// per-chunk work, not by the latency of these loads.
constexpr int GLU_SETS = 2;
struct GluBwdState {
    int chunk = 0;               // chunks this warp has been through (selects the box set and the barrier parity)
    int ahead_tile = 0, ahead_c = 0, issued = 0;   // next chunk whose gate / up boxes have not been requested yet
};
// Requests the boxes of the next not-yet-requested chunk (one lane calls this).  Tiles of this cluster are
// first_tile, first_tile + tile_step, ...; a tile has up to four 64-column chunks.
__device__ __forceinline__ void glu_bwd_prefetch(const GemmParams& p, const CUtensorMap* map_gu, uint8_t* boxes, uint64_t* bars, int q, int rank,
                                                 int tile_step, int num_tiles, GluBwdState& st) {
    using namespace ptx;
    if (st.ahead_tile >= num_tiles) return;
    const int t2 = st.ahead_tile % p.tiles_mn;
    const int row0 = tile_m(t2, p) * 256 + rank * 128 + q * 32, n0 = tile_n(t2, p) * 256;
    const int set = st.issued % GLU_SETS;
    uint8_t* g = boxes + ((q * GLU_SETS + set) * 2 + 0) * EPI_BOX_BYTES;
    uint64_t* bar = bars + q * GLU_SETS + set;
    mbar_arrive_expect_tx(bar, 2 * EPI_BOX_BYTES);
    tma_load_2d(g, map_gu, bar, n0 + st.ahead_c, row0);
    tma_load_2d(g + EPI_BOX_BYTES, map_gu, bar, p.glu_inter + n0 + st.ahead_c, row0);
    ++st.issued;
    st.ahead_c += 64;
    if (st.ahead_c >= 256 || n0 + st.ahead_c >= p.n) { st.ahead_c = 0; st.ahead_tile += tile_step; }
}
// One tile.  Returns false when a wait ran out.
__device__ __forceinline__ bool epilogue_glu_bwd(const GemmParams& p, const CUtensorMap* map_d, const CUtensorMap* map_gu, uint8_t* boxes, uint64_t* bars,
                                                 volatile int* abort_flag, uint32_t taddr, int q, int lane, int rank, int store_row0, int n0,
                                                 int tile_step, int num_tiles, GluBwdState& st, BoxPair& bp) {
    using namespace ptx;
    const bool geglu = p.glu_geglu != 0;
#pragma unroll 1
    for (int c = 0; c < 256; c += 64) {
        if (n0 + c >= p.n) break;            // uniform across the warp (inter is a multiple of 64)
        const int set = st.chunk % GLU_SETS;
        // the next request goes into the set of the previous chunk, whose stores (the latest commit) must have read it
        if (bp.side != 1 && lane == 0) {     // the helper issues neither loads nor stores
            tma_store_wait_read<0>();
            glu_bwd_prefetch(p, map_gu, boxes, bars, q, rank, tile_step, num_tiles, st);
        }
        if (!__all_sync(0xffffffffu, mbar_wait(bars + q * GLU_SETS + set, (uint32_t)((st.chunk / GLU_SETS) & 1), abort_flag))) return false;
        uint8_t* gbox = boxes + ((q * GLU_SETS + set) * 2 + 0) * EPI_BOX_BYTES;
        const uint32_t g_addr = smem_u32(gbox) + (uint32_t)lane * 128u, u_addr = g_addr + EPI_BOX_BYTES;
        for (int half = bp.half_begin(); half < bp.half_end(); ++half) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + (uint32_t)(c + half * 32), r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pos = (uint32_t)((half * 4 + j) ^ (lane & 7)) * 16u;
                uint32_t gw[4], uw[4];
                ld_shared_v4(g_addr + pos, gw[0], gw[1], gw[2], gw[3]);
                ld_shared_v4(u_addr + pos, uw[0], uw[1], uw[2], uw[3]);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[w]));
                    const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[w]));
                    const float d0 = round_bf16(__uint_as_float(r[8 * j + 2 * w]) * p.alpha), d1 = round_bf16(__uint_as_float(r[8 * j + 2 * w + 1]) * p.alpha);
                    float dg0, du0, dg1, du1;
                    glu_bwd(geglu, d0, g2.x, u2.x, dg0, du0);
                    glu_bwd(geglu, d1, g2.y, u2.y, dg1, du1);
                    const __nv_bfloat162 og = __floats2bfloat162_rn(dg0, dg1), ou = __floats2bfloat162_rn(du0, du1);
                    gw[w] = *reinterpret_cast<const uint32_t*>(&og);
                    uw[w] = *reinterpret_cast<const uint32_t*>(&ou);
                }
                st_shared_v4(g_addr + pos, gw[0], gw[1], gw[2], gw[3]);
                st_shared_v4(u_addr + pos, uw[0], uw[1], uw[2], uw[3]);
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (bp.side == 1) {
            // Nothing else holds the helper back here (its boxes arrive by TMA, not from the owner), and a parity wait
            // tells phases apart only one phase deep: the helper reports chunk k only after the owner has taken its
            // report of chunk k - 1.
            if (st.chunk > 0 && !__all_sync(0xffffffffu, mbar_wait(bp.free_bar, (uint32_t)((st.chunk - 1) & 1), abort_flag))) return false;
            if (lane == 0) mbar_arrive(bp.filled_bar);
        } else {
            if (bp.side == 0 && !__all_sync(0xffffffffu, mbar_wait(bp.filled_bar, (uint32_t)(st.chunk & 1), abort_flag))) return false;
            if (lane == 0) {
                tma_store_2d(map_d, gbox, n0 + c, store_row0);
                tma_store_2d(map_d, gbox + EPI_BOX_BYTES, p.glu_inter + n0 + c, store_row0);
                tma_store_commit();
                if (bp.side == 0) mbar_arrive(bp.free_bar);
            }
        }
        ++st.chunk;
    }
    return true;
}

// f32 outputs: boxes of 32 rows x 32 columns (128-byte rows, same swizzle), written with a tensor store or,
// when D already holds a partial result (accumulate / K split), added to memory by a tensor reduction.
template <int BN>
__device__ __forceinline__ bool epilogue_f32_tma(const GemmParams& p, const CUtensorMap* map_d, uint8_t* store_smem, uint32_t taddr,
                                                 int q, int lane, int store_row0, int n0, bool add_bias, int& box_ctr, BoxPair& bp) {
    using namespace ptx;
    bool ok = true;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.n) break;          // uniform across the warp
        uint8_t* buf = store_smem + (q * 2 + (box_ctr & 1)) * EPI_BOX_BYTES;
        const uint32_t buf_addr = smem_u32(buf) + (uint32_t)lane * 128u;
        if (!box_acquire<1>(bp, lane)) return false;
        for (int half = bp.half_begin(); half < bp.half_end(); ++half) {     // 16 of the box's 32 columns
            uint32_t r[16];
            tmem_ld_32x16(taddr + (uint32_t)(c + half * 16), r);
            tmem_ld_wait();
            const int col0 = n0 + c + half * 16;
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * p.alpha);
            if (add_bias) {
#pragma unroll
                for (int j = 0; j < 16; ++j) if (col0 + j < p.n) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(p.bias + col0 + j));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pos = (uint32_t)((half * 4 + j) ^ (lane & 7));   // 128-byte swizzle
                st_shared_v4(buf_addr + pos * 16u, r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
        }
        if (box_release(bp, lane, ok) && lane == 0) {
            if (p.f32_reduce) tma_reduce_add_2d(map_d, buf, n0 + c, store_row0);
            else tma_store_2d(map_d, buf, n0 + c, store_row0);
            tma_store_commit();
        }
        if (!ok) return false;
        ++box_ctr;
    }
    return true;
}

}  // namespace mft
