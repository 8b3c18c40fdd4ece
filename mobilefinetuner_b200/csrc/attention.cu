// Fused causal / sliding-window GQA attention, forward and backward.
//
// Replaces the reference's materialised chain repeat_kv_heads -> transpose ->
// matmul -> mul(scale) -> add(mask) -> softmax -> matmul and its autograd
// (four [B,nh,S,S] fp32 tensors forward, as many backward) by flash-style
// kernels that keep scores on chip:
//   forward : one CTA per (BM queries, head, batch); online softmax in fp32
//             (exp2 domain); masks are index predicates, fully masked key
//             blocks are skipped; writes O (bf16) and the row log-sum-exp.
//   backward: delta = rowsum(O * dO); a query-stationary kernel for dQ and a
//             key-stationary kernel for dK/dV, both recomputing P from the
//             saved log-sum-exp.  The key-stationary kernel either loops over
//             the query heads of a KV group (dK/dV come out per KV head with
//             no repeat_kv copy and no atomics) or, given an fp32 scratch,
//             runs one CTA per query head and adds into the scratch (4x the
//             CTAs for a 4:1 group; a small kernel converts to bf16).
// All three stream their moving tiles through a two-stage cp.async ring: the
// loads of tile t+1 are in flight while tile t is multiplied.
// Query head h uses KV head h / (n_heads / n_kv_heads).
// Tensor-core path: warp-level mma.sync m16n8k16 (bf16 in, fp32 accumulate).
#include "common.cuh"

#include <cstdlib>

#include "attention.h"

namespace mft {

namespace {

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16z(void* smem, const void* gmem, bool valid) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async4z(void* smem, const void* gmem, bool valid) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


// Copy a [ROWS x HD] bf16 tile (row r at g + r*stride, rows >= rows_valid zero-filled)
// into shared memory with padded row stride HD+8.
template <int ROWS, int HD, int THREADS>
__device__ __forceinline__ void load_tile(__nv_bfloat16* s, const __nv_bfloat16* g, int64_t stride, int rows_valid) {
    constexpr int VPR = HD / 8;
    for (int i = threadIdx.x; i < ROWS * VPR; i += THREADS) {
        const int r = i / VPR, c = (i % VPR) * 8;
        const bool ok = r < rows_valid;
        cp_async16z(s + r * (HD + 8) + c, ok ? g + (int64_t)r * stride + c : g, ok);
    }
}

// acc[nb] (16 x 8*NB slab) = A[16 rows of `a_s`] * B^T where both tiles
// are stored [row][HD] (contraction along HD): S = Q K^T, dP = dO V^T.
template <int HD, int NB>
__device__ __forceinline__ void mma_rowrow(float (&acc)[NB][4], const __nv_bfloat16* a_s, int a_row0,
                                           const __nv_bfloat16* b_s, int lane) {
    constexpr int LD = HD + 8;
#pragma unroll
    for (int kk = 0; kk < HD; kk += 16) {
        uint32_t a[4];
        ldsm_x4(a, a_s + (a_row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk + (lane >> 4) * 8);
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
            uint32_t b[4];
            ldsm_x4(b, b_s + (nb * 8 + (lane & 7) + (lane >> 4) * 8) * LD + kk + ((lane >> 3) & 1) * 8);
            mma16816(acc[nb], a, b[0], b[1]);
            mma16816(acc[nb + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ bool visible(int i, int j, int seq, int window) {
    return j <= i && j < seq && (window <= 0 || i - j < window);
}

// ---------------------------------------------------------------- forward
// BM queries per CTA (one warp per 16), BN keys per tile.
template <int HD, int BM, int BN, int STAGES>
__global__ void __launch_bounds__(BM * 2)
attn_fwd_kernel(const AttnParams p) {
    dep_trigger();
    dep_wait();
    constexpr int LD = HD + 8, THREADS = BM * 2, NB = BN / 8;
    extern __shared__ __align__(16) uint8_t smem_attn[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_attn);
    __nv_bfloat16* KV = Qs + BM * LD;             // 2 stages of { K [BN][LD], V [BN][LD] }
    const int qb = gridDim.x - 1 - blockIdx.x;   // longest rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.rep;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int i0 = qb * BM;
    const int rows_q = min(BM, p.seq - i0);
    const __nv_bfloat16* kbase = p.k + (int64_t)b * p.sk.stride_b + (int64_t)kvh * p.sk.stride_h;
    const __nv_bfloat16* vbase = p.v + (int64_t)b * p.sv.stride_b + (int64_t)kvh * p.sv.stride_h;
    auto prefetch = [&](int jb, int st) {
        const int j0 = jb * BN, rows_k = min(BN, p.seq - j0);
        __nv_bfloat16* Ks = KV + st * 2 * BN * LD;
        load_tile<BN, HD, THREADS>(Ks, kbase + (int64_t)j0 * p.sk.stride_s, p.sk.stride_s, rows_k);
        load_tile<BN, HD, THREADS>(Ks + BN * LD, vbase + (int64_t)j0 * p.sv.stride_s, p.sv.stride_s, rows_k);
        cp_commit();
    };

    const int i_last = min(i0 + BM - 1, p.seq - 1);
    const int jb_hi = i_last / BN;
    const int jb_lo = p.window > 0 ? max(0, i0 - p.window + 1) / BN : 0;
    const float sl2 = p.scale * LOG2E;
    load_tile<BM, HD, THREADS>(Qs, p.q + (int64_t)b * p.sq.stride_b + (int64_t)i0 * p.sq.stride_s + (int64_t)h * p.sq.stride_h, p.sq.stride_s, rows_q);
    prefetch(jb_lo, 0);

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_a = i0 + warp * 16 + g;       // rows of c0,c1 ; c2,c3 belong to row_a + 8

    for (int jb = jb_lo; jb <= jb_hi; ++jb) {
        const int j0 = jb * BN;
        const int st = STAGES == 2 ? (jb - jb_lo) & 1 : 0;
        if (STAGES == 1 && jb > jb_lo) {
            __syncthreads();   // everyone is done with the single stage
            prefetch(jb, 0);
        }
        cp_wait_all();
        __syncthreads();   // tile jb has landed; with two stages everyone is also done with the other one
        if (STAGES == 2 && jb < jb_hi) prefetch(jb + 1, st ^ 1);
        const __nv_bfloat16* Ks = KV + st * 2 * BN * LD;
        const __nv_bfloat16* Vs = Ks + BN * LD;

        float s[NB][4];
#pragma unroll
        for (int i = 0; i < NB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
        mma_rowrow<HD, NB>(s, Qs, warp * 16, Ks, lane);

        const bool need_mask = (j0 + BN - 1 > i0) || (j0 + BN > p.seq) ||
                               (p.window > 0 && j0 < i0 + BM - p.window);
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row_a + (e >> 1) * 8, j = j0 + nb * 8 + tq * 2 + (e & 1);
                float val = s[nb][e] * sl2;
                if (need_mask && !visible(i, j, p.seq, p.window)) val = -INFINITY;
                s[nb][e] = val;
                m_new[e >> 1] = fmaxf(m_new[e >> 1], val);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
        }
        float corr[2], m_use[2], l_add[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_use[r] = (m_new[r] == -INFINITY) ? 0.f : m_new[r];
            corr[r] = exp2f(m_run[r] - m_use[r]);     // m_run = -inf -> 0
            m_run[r] = m_new[r];
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nb][e] - m_use[e >> 1]);
                s[nb][e] = pv;
                l_add[e >> 1] += pv;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + l_add[r];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }

        // O += P V : P from registers (bf16), V tile [key][d] via transposing ldmatrix
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int db = 0; db < HD / 8; db += 2) {
                uint32_t bb[4];
                ldsm_x4_t(bb, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + db * 8 + (lane >> 4) * 8);
                mma16816(o[db], a, bb[0], bb[1]);
                mma16816(o[db + 1], a, bb[2], bb[3]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = row_a + r * 8;
        if (i < p.seq) {
            const float inv = l_run[r] > 0.f ? 1.0f / l_run[r] : 0.f;
            __nv_bfloat16* orow = p.out + (int64_t)b * p.so.stride_b + (int64_t)i * p.so.stride_s + (int64_t)h * p.so.stride_h;
#pragma unroll
            for (int db = 0; db < HD / 8; ++db) {
                *reinterpret_cast<uint32_t*>(orow + db * 8 + tq * 2) = pack_bf16(o[db][r * 2] * inv, o[db][r * 2 + 1] * inv);
            }
            if (tq == 0) p.lse[((int64_t)b * p.n_heads + h) * p.seq + i] = (m_run[r] + log2f(l_run[r])) / LOG2E;
        }
    }
}

// ---------------------------------------------------------------- backward: delta
// delta[b,h,i] = sum_d O[i,d] * dO[i,d]; one warp per row.
template <int HD>
__global__ void attn_delta_kernel(const AttnParams p) {
    dep_trigger();
    dep_wait();
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t total = (int64_t)p.batch * p.n_heads * p.seq;
    if (wid >= total) return;
    const int i = (int)(wid % p.seq), h = (int)((wid / p.seq) % p.n_heads), b = (int)(wid / ((int64_t)p.seq * p.n_heads));
    const __nv_bfloat16* orow = p.o + (int64_t)b * p.so.stride_b + (int64_t)i * p.so.stride_s + (int64_t)h * p.so.stride_h;
    const __nv_bfloat16* drow = p.d_o + (int64_t)b * p.sdo.stride_b + (int64_t)i * p.sdo.stride_s + (int64_t)h * p.sdo.stride_h;
    float acc = 0.f;
    if (HD >= 256 && ((reinterpret_cast<uintptr_t>(orow) | reinterpret_cast<uintptr_t>(drow)) & 15) == 0) {
        // 16-byte accesses: one per operand and lane at head_dim 256
        for (int d = lane * 8; d < HD; d += 256) {
            const uint4 a4 = *reinterpret_cast<const uint4*>(orow + d), c4 = *reinterpret_cast<const uint4*>(drow + d);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a4);
            const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = __bfloat1622float2(a2[j]), c = __bfloat1622float2(c2[j]);
                acc += a.x * c.x + a.y * c.y;
            }
        }
    } else {
        for (int d = lane * 2; d < HD; d += 64) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(orow + d));
            const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(drow + d));
            acc += a.x * c.x + a.y * c.y;
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) p.delta[wid] = acc;
}

// ---------------------------------------------------------------- backward: dQ (query-stationary)
template <int HD, int BM, int BN, int STAGES>
__global__ void __launch_bounds__(BM * 2)
attn_bwd_dq_kernel(const AttnParams p) {
    dep_trigger();
    dep_wait();
    constexpr int LD = HD + 8, THREADS = BM * 2, NB = BN / 8;
    extern __shared__ __align__(16) uint8_t smem_attn[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_attn);
    __nv_bfloat16* dOs = Qs + BM * LD;
    __nv_bfloat16* KV = dOs + BM * LD;            // 2 stages of { K [BN][LD], V [BN][LD] }
    const int qb = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.rep;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int i0 = qb * BM;
    const int rows_q = min(BM, p.seq - i0);
    const __nv_bfloat16* kbase = p.k + (int64_t)b * p.sk.stride_b + (int64_t)kvh * p.sk.stride_h;
    const __nv_bfloat16* vbase = p.v + (int64_t)b * p.sv.stride_b + (int64_t)kvh * p.sv.stride_h;
    auto prefetch = [&](int jb, int st) {
        const int j0 = jb * BN, rows_k = min(BN, p.seq - j0);
        __nv_bfloat16* Ks = KV + st * 2 * BN * LD;
        load_tile<BN, HD, THREADS>(Ks, kbase + (int64_t)j0 * p.sk.stride_s, p.sk.stride_s, rows_k);
        load_tile<BN, HD, THREADS>(Ks + BN * LD, vbase + (int64_t)j0 * p.sv.stride_s, p.sv.stride_s, rows_k);
        cp_commit();
    };
    const int i_last = min(i0 + BM - 1, p.seq - 1);
    const int jb_hi = i_last / BN;
    const int jb_lo = p.window > 0 ? max(0, i0 - p.window + 1) / BN : 0;
    load_tile<BM, HD, THREADS>(Qs, p.q + (int64_t)b * p.sq.stride_b + (int64_t)i0 * p.sq.stride_s + (int64_t)h * p.sq.stride_h, p.sq.stride_s, rows_q);
    load_tile<BM, HD, THREADS>(dOs, p.d_o + (int64_t)b * p.sdo.stride_b + (int64_t)i0 * p.sdo.stride_s + (int64_t)h * p.sdo.stride_h, p.sdo.stride_s, rows_q);
    prefetch(jb_lo, 0);

    const float sl2 = p.scale * LOG2E;
    const int row_a = i0 + warp * 16 + g;
    float lse2[2], dlt[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = row_a + r * 8;
        const bool ok = i < p.seq;
        const int64_t idx = ((int64_t)b * p.n_heads + h) * p.seq + (ok ? i : 0);
        lse2[r] = ok ? p.lse[idx] * LOG2E : 0.f;
        dlt[r] = ok ? p.delta[idx] : 0.f;
    }
    float dq[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }

    for (int jb = jb_lo; jb <= jb_hi; ++jb) {
        const int j0 = jb * BN;
        const int st = STAGES == 2 ? (jb - jb_lo) & 1 : 0;
        if (STAGES == 1 && jb > jb_lo) {
            __syncthreads();   // everyone is done with the single stage
            prefetch(jb, 0);
        }
        cp_wait_all();
        __syncthreads();   // tile jb has landed; with two stages everyone is also done with the other one
        if (STAGES == 2 && jb < jb_hi) prefetch(jb + 1, st ^ 1);
        const __nv_bfloat16* Ks = KV + st * 2 * BN * LD;
        const __nv_bfloat16* Vs = Ks + BN * LD;
        float s[NB][4], dp[NB][4];
#pragma unroll
        for (int i = 0; i < NB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f; }
        mma_rowrow<HD, NB>(s, Qs, warp * 16, Ks, lane);
        mma_rowrow<HD, NB>(dp, dOs, warp * 16, Vs, lane);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row_a + (e >> 1) * 8, j = j0 + nb * 8 + tq * 2 + (e & 1);
                const bool vis = i < p.seq && visible(i, j, p.seq, p.window);
                const float pv = vis ? exp2f(s[nb][e] * sl2 - lse2[e >> 1]) : 0.f;
                s[nb][e] = pv * (dp[nb][e] - dlt[e >> 1]);     // dS (without the softmax scale)
            }
        // dQ += dS K : K tile [key][d] as the [k][n] operand via transposing ldmatrix
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int db = 0; db < HD / 8; db += 2) {
                uint32_t bb[4];
                ldsm_x4_t(bb, Ks + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + db * 8 + (lane >> 4) * 8);
                mma16816(dq[db], a, bb[0], bb[1]);
                mma16816(dq[db + 1], a, bb[2], bb[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = row_a + r * 8;
        if (i < p.seq) {
            __nv_bfloat16* row = p.dq + (int64_t)b * p.sq.stride_b + (int64_t)i * p.sq.stride_s + (int64_t)h * p.sq.stride_h;
#pragma unroll
            for (int db = 0; db < HD / 8; ++db)
                *reinterpret_cast<uint32_t*>(row + db * 8 + tq * 2) = pack_bf16(dq[db][r * 2] * p.scale, dq[db][r * 2 + 1] * p.scale);
        }
    }
}

// ---------------------------------------------------------------- backward: dK, dV (key-stationary)
// 4 x WN warps: warp (wm, wn) owns keys 16*wm..+15 and the d-columns
// [wn*HD/WN, (wn+1)*HD/WN).  S^T and dP^T (keys x queries) are computed with the
// 64 queries split across the WN warps of a row, written to shared memory as
// bf16 and re-read as the A operand of the two accumulating products.
// SPLIT = false: grid.y = KV heads, the CTA walks all query heads of its group and stores bf16 dK/dV.
// SPLIT = true : grid.y = query heads, the CTA adds its head's contribution into the f32 accumulator.
template <int HD, int WN, bool SPLIT>
__global__ void __launch_bounds__(128 * WN)
attn_bwd_dkv_kernel(const AttnParams p) {
    dep_trigger();
    dep_wait();
    constexpr int BM = 64, BN = 64;
    constexpr int LD = HD + 8;
    constexpr int THREADS = 128 * WN;
    constexpr int PLD = BM + 8;            // row stride of the P^T / dS^T tiles
    constexpr int DW = HD / WN;            // d-columns per warp
    constexpr int QW = BM / WN;            // queries per warp in the score products
    constexpr int STAGE = 2 * BM * LD;     // elements of one { Q, dO } stage
    extern __shared__ __align__(16) uint8_t smem_attn[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_attn);
    __nv_bfloat16* Vs = Ks + BN * LD;
    __nv_bfloat16* QdO = Vs + BN * LD;                       // 2 stages of { Q [BM][LD], dO [BM][LD] }
    __nv_bfloat16* Pt = QdO + 2 * STAGE;                     // [64 keys][PLD]
    __nv_bfloat16* dSt = Pt + BN * PLD;
    float* stats = reinterpret_cast<float*>(dSt + BN * PLD);  // 2 stages of { lse [BM], delta [BM] }

    const int jb = blockIdx.x, b = blockIdx.z;
    const int kvh = SPLIT ? blockIdx.y / p.rep : blockIdx.y;
    const int h_first = SPLIT ? blockIdx.y : kvh * p.rep;
    const int n_heads_here = SPLIT ? 1 : p.rep;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp % 4, wn = warp / 4;
    const int g = lane >> 2, tq = lane & 3;
    const int j0 = jb * BN;
    const int rows_k = min(BN, p.seq - j0);
    load_tile<BN, HD, THREADS>(Ks, p.k + (int64_t)b * p.sk.stride_b + (int64_t)j0 * p.sk.stride_s + (int64_t)kvh * p.sk.stride_h, p.sk.stride_s, rows_k);
    load_tile<BN, HD, THREADS>(Vs, p.v + (int64_t)b * p.sv.stride_b + (int64_t)j0 * p.sv.stride_s + (int64_t)kvh * p.sv.stride_h, p.sv.stride_s, rows_k);

    // queries that can see keys j0 .. j0+63: i >= j0 and i - j < window
    const int i_max = p.window > 0 ? min(p.seq - 1, j0 + BN - 1 + p.window - 1) : p.seq - 1;
    const int qb_lo = j0 / BM, qb_hi = i_max / BM;
    const int nq = qb_hi - qb_lo + 1, n_it = nq * n_heads_here;
    const float sl2 = p.scale * LOG2E;
    auto prefetch = [&](int it, int st) {
        const int h = h_first + it / nq, i0 = (qb_lo + it % nq) * BM;
        const int rows_q = min(BM, p.seq - i0);
        __nv_bfloat16* Qs = QdO + st * STAGE;
        load_tile<BM, HD, THREADS>(Qs, p.q + (int64_t)b * p.sq.stride_b + (int64_t)i0 * p.sq.stride_s + (int64_t)h * p.sq.stride_h, p.sq.stride_s, rows_q);
        load_tile<BM, HD, THREADS>(Qs + BM * LD, p.d_o + (int64_t)b * p.sdo.stride_b + (int64_t)i0 * p.sdo.stride_s + (int64_t)h * p.sdo.stride_h, p.sdo.stride_s, rows_q);
        if (threadIdx.x < 2 * BM) {
            const int r = threadIdx.x % BM;
            const bool ok = i0 + r < p.seq;
            const int64_t idx = ((int64_t)b * p.n_heads + h) * p.seq + (ok ? i0 + r : 0);
            cp_async4z(stats + st * 2 * BM + threadIdx.x, (threadIdx.x < BM ? p.lse : p.delta) + idx, ok);
        }
        cp_commit();
    };
    prefetch(0, 0);

    float dk[DW / 8][4], dv[DW / 8][4];
#pragma unroll
    for (int i = 0; i < DW / 8; ++i) { dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f; dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f; }

    for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const int i0 = (qb_lo + it % nq) * BM;
        cp_wait_all();
        __syncthreads();     // stage `st` has landed; everyone is done with the other stage and with Pt / dSt
        if (it + 1 < n_it) prefetch(it + 1, st ^ 1);
        const __nv_bfloat16* Qs = QdO + st * STAGE;
        const __nv_bfloat16* dOs = Qs + BM * LD;
        const float* lse_s = stats + st * 2 * BM;
        const float* dlt_s = lse_s + BM;

        // S^T[key, query] and dP^T[key, query] for this warp's 16 keys x QW queries
        float st_[QW / 8][4], dpt[QW / 8][4];
#pragma unroll
        for (int i = 0; i < QW / 8; ++i) { st_[i][0] = st_[i][1] = st_[i][2] = st_[i][3] = 0.f; dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD; kk += 16) {
            uint32_t ak[4], av[4];
            const int arow = wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldsm_x4(ak, Ks + arow * LD + kk + (lane >> 4) * 8);
            ldsm_x4(av, Vs + arow * LD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < QW / 8; nb += 2) {
                uint32_t bq[4], bd[4];
                const int brow = wn * QW + nb * 8 + (lane & 7) + (lane >> 4) * 8;
                ldsm_x4(bq, Qs + brow * LD + kk + ((lane >> 3) & 1) * 8);
                ldsm_x4(bd, dOs + brow * LD + kk + ((lane >> 3) & 1) * 8);
                mma16816(st_[nb], ak, bq[0], bq[1]);
                mma16816(st_[nb + 1], ak, bq[2], bq[3]);
                mma16816(dpt[nb], av, bd[0], bd[1]);
                mma16816(dpt[nb + 1], av, bd[2], bd[3]);
            }
        }
#pragma unroll
        for (int nb = 0; nb < QW / 8; ++nb)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const int jl = wm * 16 + g + (e >> 1) * 8;          // key within tile
                const int il = wn * QW + nb * 8 + tq * 2;            // query within tile
                float pv[2], ds[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int i = i0 + il + c, j = j0 + jl;
                    const bool vis = i < p.seq && visible(i, j, p.seq, p.window);
                    pv[c] = vis ? exp2f(st_[nb][e + c] * sl2 - lse_s[il + c] * LOG2E) : 0.f;
                    ds[c] = pv[c] * (dpt[nb][e + c] - dlt_s[il + c]);
                }
                *reinterpret_cast<uint32_t*>(Pt + jl * PLD + il) = pack_bf16(pv[0], pv[1]);
                *reinterpret_cast<uint32_t*>(dSt + jl * PLD + il) = pack_bf16(ds[0], ds[1]);
            }
        __syncthreads();
        // dV += P^T dO ; dK += dS^T Q  (contraction over the 64 queries)
#pragma unroll
        for (int kk = 0; kk < BM; kk += 16) {
            uint32_t ap[4], ad[4];
            const int arow = wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldsm_x4(ap, Pt + arow * PLD + kk + (lane >> 4) * 8);
            ldsm_x4(ad, dSt + arow * PLD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int db = 0; db < DW / 8; db += 2) {
                uint32_t b1[4], b2[4];
                const int brow = kk + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int bcol = wn * DW + db * 8 + (lane >> 4) * 8;
                ldsm_x4_t(b1, dOs + brow * LD + bcol);
                ldsm_x4_t(b2, Qs + brow * LD + bcol);
                mma16816(dv[db], ap, b1[0], b1[1]);
                mma16816(dv[db + 1], ap, b1[2], b1[3]);
                mma16816(dk[db], ad, b2[0], b2[1]);
                mma16816(dk[db + 1], ad, b2[2], b2[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = j0 + wm * 16 + g + r * 8;
        if (j < p.seq) {
            if constexpr (SPLIT) {
                const int64_t half = (int64_t)p.batch * p.seq * p.n_kv * HD;
                float* krow = p.dkv_acc + (((int64_t)b * p.seq + j) * p.n_kv + kvh) * HD + wn * DW;
                float* vrow = krow + half;
#pragma unroll
                for (int db = 0; db < DW / 8; ++db) {
                    atomicAdd(krow + db * 8 + tq * 2, dk[db][r * 2] * p.scale);
                    atomicAdd(krow + db * 8 + tq * 2 + 1, dk[db][r * 2 + 1] * p.scale);
                    atomicAdd(vrow + db * 8 + tq * 2, dv[db][r * 2]);
                    atomicAdd(vrow + db * 8 + tq * 2 + 1, dv[db][r * 2 + 1]);
                }
            } else {
                __nv_bfloat16* krow = p.dk + (int64_t)b * p.sk.stride_b + (int64_t)j * p.sk.stride_s + (int64_t)kvh * p.sk.stride_h + wn * DW;
                __nv_bfloat16* vrow = p.dv + (int64_t)b * p.sv.stride_b + (int64_t)j * p.sv.stride_s + (int64_t)kvh * p.sv.stride_h + wn * DW;
#pragma unroll
                for (int db = 0; db < DW / 8; ++db) {
                    *reinterpret_cast<uint32_t*>(krow + db * 8 + tq * 2) = pack_bf16(dk[db][r * 2] * p.scale, dk[db][r * 2 + 1] * p.scale);
                    *reinterpret_cast<uint32_t*>(vrow + db * 8 + tq * 2) = pack_bf16(dv[db][r * 2], dv[db][r * 2 + 1]);
                }
            }
        }
    }
}

// f32 accumulator [2][batch, seq, n_kv, HD] -> bf16 dK / dV with the caller's strides
template <int HD>
__global__ void attn_dkv_store_kernel(const AttnParams p) {
    dep_trigger();
    dep_wait();
    const int64_t half = (int64_t)p.batch * p.seq * p.n_kv * HD;
    const int64_t total = 2 * half / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = i * 4;
        const bool is_v = e >= half;
        const int64_t r = is_v ? e - half : e;
        const int d = (int)(r % HD), kvh = (int)((r / HD) % p.n_kv);
        const int64_t tok = r / ((int64_t)HD * p.n_kv);
        const int j = (int)(tok % p.seq), b = (int)(tok / p.seq);
        const float4 a = *reinterpret_cast<const float4*>(p.dkv_acc + e);
        const mft_strides_t& ss = is_v ? p.sv : p.sk;
        __nv_bfloat16* out = (is_v ? p.dv : p.dk) + (int64_t)b * ss.stride_b + (int64_t)j * ss.stride_s + (int64_t)kvh * ss.stride_h + d;
        *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
    }
}

// MFT_ATTN_SHAPE selects an alternative tile shape of the head_dim 256 kernels (tuning aid; 0 = default).
int attn_shape_override() {
    static const int v = [] { const char* e = std::getenv("MFT_ATTN_SHAPE"); return e ? std::atoi(e) : 0; }();
    return v;
}

template <typename K>
int32_t set_smem(K kernel, int bytes) {
    return check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "attention smem attribute");
}

int32_t check_common(const AttnParams& p, int64_t hd) {
    if (!(hd == 64 || hd == 128 || hd == 256)) return fail(MFT_ERR_UNSUPPORTED, "attention: head_dim must be 64, 128 or 256");
    if (p.n_heads % p.n_kv != 0) return fail(MFT_ERR_INVALID_ARG, "attention: n_heads must be a multiple of n_kv_heads");
    const mft_strides_t* ss[5] = {&p.sq, &p.sk, &p.sv, &p.so, &p.sdo};
    for (auto s : ss)
        if (s->stride_b % 8 || s->stride_s % 8 || s->stride_h % 8) return fail(MFT_ERR_INVALID_ARG, "attention: strides must be multiples of 8 elements");
    return MFT_OK;
}

}  // namespace
}  // namespace mft

using namespace mft;

extern "C" int32_t mft_attn_fwd(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk, const void* v,
                                mft_strides_t sv, void* o, mft_strides_t so, float* lse, int64_t batch, int64_t seq,
                                int64_t n_heads, int64_t n_kv, int64_t hd, float scale, int64_t window, mft_stream_t stream) {
    MFT_CHECK_ARG(q && k && v && o && lse && batch > 0 && seq > 0 && n_heads > 0 && n_kv > 0, "mft_attn_fwd: bad argument");
    MFT_CHECK_ARG(batch <= 65535 && n_heads <= 65535, "mft_attn_fwd: batch / heads too large");
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.out = (__nv_bfloat16*)o;
    p.lse = lse; p.sq = sq; p.sk = sk; p.sv = sv; p.so = so; p.sdo = so;
    p.batch = (int)batch; p.seq = (int)seq; p.n_heads = (int)n_heads; p.n_kv = (int)n_kv; p.rep = (int)(n_heads / n_kv);
    p.scale = scale; p.window = (int)window;
    MFT_CHECK_ARG(seq <= 65535 || (hd == 64 || hd == 128 || hd == 256), "mft_attn_fwd: sequence too long for this head_dim");
    if (!(hd == 64 || hd == 128 || hd == 256)) return attn_generic_fwd(p, (int)hd, as_stream(stream));
    if (int32_t s = check_common(p, hd)) return s;
    {   // tcgen05 kernel when the problem qualifies
        const int32_t s2 = attn_fwd_sm100(p, (int)hd, as_stream(stream));
        if (s2 != MFT_ERR_UNSUPPORTED) return s2;
    }
#define FWD(HD, BM, BN, ST)                                                                  \
    {                                                                                        \
        dim3 grid((unsigned)((seq + BM - 1) / BM), (unsigned)n_heads, (unsigned)batch);      \
        const int bytes = (BM + 2 * ST * BN) * (HD + 8) * 2;                                 \
        if (int32_t s = set_smem(attn_fwd_kernel<HD, BM, BN, ST>, bytes)) return s;          \
        launch_dep(attn_fwd_kernel<HD, BM, BN, ST>, dim3(grid), dim3(BM * 2), (size_t)(bytes), as_stream(stream), p);      \
    }
    const int shape = attn_shape_override();
    // measured best on B200: 64-query CTAs (two resident per SM) beat 128-query ones; at head_dim 256 the
    // second stage costs a resident CTA and loses
    if (hd == 64) { if (shape == 1) FWD(64, 128, 64, 2) else FWD(64, 64, 64, 2) }
    else if (hd == 128) { if (shape == 1) FWD(128, 128, 64, 2) else FWD(128, 64, 64, 2) }
    else if (shape == 1) FWD(256, 128, 64, 2) else if (shape == 2) FWD(256, 64, 32, 2) else FWD(256, 64, 64, 1)
#undef FWD
    MFT_LAUNCH_CHECK("attn_fwd");
    return MFT_OK;
}

extern "C" int32_t mft_attn_bwd(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk, const void* v,
                                mft_strides_t sv, const void* o, mft_strides_t so, const void* d_o, mft_strides_t sdo,
                                const float* lse, void* dq, void* dk, void* dv, float* delta, float* dkv_acc, int64_t batch,
                                int64_t seq, int64_t n_heads, int64_t n_kv, int64_t hd, float scale, int64_t window,
                                mft_stream_t stream) {
    MFT_CHECK_ARG(q && k && v && o && d_o && lse && dq && dk && dv && delta, "mft_attn_bwd: null pointer");
    MFT_CHECK_ARG(batch > 0 && seq > 0 && n_heads > 0 && n_kv > 0 && batch <= 65535 && n_heads <= 65535, "mft_attn_bwd: bad size");
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.o = (const __nv_bfloat16*)o; p.d_o = (const __nv_bfloat16*)d_o;
    p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
    p.lse = const_cast<float*>(lse); p.delta = delta; p.dkv_acc = dkv_acc;
    p.sq = sq; p.sk = sk; p.sv = sv; p.so = so; p.sdo = sdo;
    p.batch = (int)batch; p.seq = (int)seq; p.n_heads = (int)n_heads; p.n_kv = (int)n_kv; p.rep = (int)(n_heads / n_kv);
    p.scale = scale; p.window = (int)window;
    MFT_CHECK_ARG(seq <= 65535 || (hd == 64 || hd == 128 || hd == 256), "mft_attn_bwd: sequence too long for this head_dim");
    if (!(hd == 64 || hd == 128 || hd == 256)) return attn_generic_bwd(p, (int)hd, as_stream(stream));
    if (int32_t s = check_common(p, hd)) return s;
    const int64_t rows = batch * n_heads * seq;
    const unsigned dblocks = (unsigned)((rows * 32 + 255) / 256);
    // dK / dV are collected in the caller's f32 scratch when it is given: by the tensor-memory kernel, or with one
    // mma.sync CTA per query head when a KV group has several heads (more, shorter CTAs)
    const int shape = attn_shape_override();
    bool dkv_tc = false;
    if (dkv_acc != nullptr)
        if (int32_t s = check_cuda(cudaMemsetAsync(dkv_acc, 0, (size_t)(2 * batch * seq * n_kv * hd) * sizeof(float), as_stream(stream)), "attention dkv memset")) return s;
    const bool split = dkv_acc != nullptr && p.rep > 1;
    dim3 gk((unsigned)((seq + 63) / 64), (unsigned)(split ? n_heads : n_kv), (unsigned)batch);
#define DQ(HD, BM, BN, ST)                                                                                  \
    {                                                                                                       \
        dim3 gq((unsigned)((seq + BM - 1) / BM), (unsigned)n_heads, (unsigned)batch);                       \
        const int b1 = (2 * BM + 2 * ST * BN) * (HD + 8) * 2;                                               \
        if (int32_t s = set_smem(attn_bwd_dq_kernel<HD, BM, BN, ST>, b1)) return s;                         \
        launch_dep(attn_bwd_dq_kernel<HD, BM, BN, ST>, dim3(gq), dim3(BM * 2), (size_t)(b1), as_stream(stream), p);                       \
        MFT_LAUNCH_CHECK("attn_bwd_dq");                                                                    \
    }
#define DKV(HD, WN, SPLIT)                                                                                  \
    {                                                                                                       \
        const int b2 = 6 * 64 * (HD + 8) * 2 + 2 * 64 * (64 + 8) * 2 + 4 * 64 * 4;                          \
        if (int32_t s = set_smem(attn_bwd_dkv_kernel<HD, WN, SPLIT>, b2)) return s;                         \
        launch_dep(attn_bwd_dkv_kernel<HD, WN, SPLIT>, dim3(gk), dim3(128 * WN), (size_t)(b2), as_stream(stream), p);                     \
        MFT_LAUNCH_CHECK("attn_bwd_dkv");                                                                   \
        if (SPLIT) {                                                                                        \
            launch_dep(attn_dkv_store_kernel<HD>, dim3(148 * 8), dim3(256), (size_t)(0), as_stream(stream), p);                           \
            MFT_LAUNCH_CHECK("attn_dkv_store");                                                             \
        }                                                                                                   \
    }
#define BWD(HD, WN, BM, BN, ST)                                                                             \
    {                                                                                                       \
        /* rowsum(O * dO) in its own kernel: forming it inside the tensor-memory dQ kernel (compute_delta) was */ \
        /* measured 0.1 ms per layer slower, it delays the start of every CTA's tile pipeline */              \
        launch_dep(attn_delta_kernel<HD>, dim3(dblocks), dim3(256), (size_t)(0), as_stream(stream), p);     \
        MFT_LAUNCH_CHECK("attn_delta");                                                                     \
        const int32_t sdq = attn_dq_sm100(p, HD, false, as_stream(stream));                                 \
        if (sdq != MFT_OK && sdq != MFT_ERR_UNSUPPORTED) return sdq;                                        \
        if (sdq == MFT_ERR_UNSUPPORTED) DQ(HD, BM, BN, ST)                                                  \
        const int32_t skv = attn_dkv_sm100(p, HD, as_stream(stream));                                       \
        if (skv != MFT_OK && skv != MFT_ERR_UNSUPPORTED) return skv;                                        \
        dkv_tc = skv == MFT_OK;                                                                             \
        if (dkv_tc) {                                                                                       \
            launch_dep(attn_dkv_store_kernel<HD>, dim3(148 * 8), dim3(256), (size_t)(0), as_stream(stream), p);                           \
            MFT_LAUNCH_CHECK("attn_dkv_store");                                                             \
        } else if (split) DKV(HD, WN, true) else DKV(HD, WN, false)                                         \
    }
    if (hd == 64) { if (shape == 1) BWD(64, 1, 128, 64, 2) else BWD(64, 1, 64, 64, 2) }
    else if (hd == 128) BWD(128, 1, 64, 64, 2)
    else if (shape == 1) BWD(256, 2, 64, 64, 2) else if (shape == 2) BWD(256, 2, 64, 32, 2) else BWD(256, 2, 64, 32, 1)
#undef DQ
#undef DKV
#undef BWD
    return MFT_OK;
}

// ---------------------------------------------------------------- allocation-free backward
// Scratch for mft_attn_bwd_noalloc: the per-row sums delta[b,h,i] = sum_d O*dO live in this
// fixed array instead of a caller-supplied buffer.  Every GPU that loads the library holds
// these 4 MiB until the process exits.
constexpr int64_t MFT_ATTN_NOALLOC_MAX_ROWS = 1 << 20;
static __device__ __align__(256) float g_attn_noalloc_delta[MFT_ATTN_NOALLOC_MAX_ROWS];

#include <mutex>

extern "C" int32_t mft_attn_bwd_noalloc(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk, const void* v,
                                        mft_strides_t sv, const void* o, mft_strides_t so, const void* d_o, mft_strides_t sdo,
                                        const float* lse, void* dq, void* dk, void* dv, int64_t batch, int64_t seq,
                                        int64_t n_heads, int64_t n_kv, int64_t hd, float scale, int64_t window,
                                        mft_stream_t stream) {
    MFT_CHECK_ARG(batch > 0 && seq > 0 && n_heads > 0, "mft_attn_bwd_noalloc: bad size");
    // each factor is bounded before the product is formed, so the product cannot wrap
    MFT_CHECK_ARG(batch <= MFT_ATTN_NOALLOC_MAX_ROWS && seq <= MFT_ATTN_NOALLOC_MAX_ROWS && n_heads <= MFT_ATTN_NOALLOC_MAX_ROWS,
                  "mft_attn_bwd_noalloc: the problem exceeds the built-in scratch; use mft_attn_bwd with a caller-supplied delta buffer");
    if (batch * n_heads > MFT_ATTN_NOALLOC_MAX_ROWS || batch * n_heads * seq > MFT_ATTN_NOALLOC_MAX_ROWS)
        return fail(MFT_ERR_INVALID_ARG, "mft_attn_bwd_noalloc: batch*n_heads*seq = " + std::to_string(batch * n_heads * seq) +
                                             " exceeds the built-in scratch of " + std::to_string(MFT_ATTN_NOALLOC_MAX_ROWS) +
                                             " rows; use mft_attn_bwd with a caller-supplied delta buffer");
    // The array's name is only a host-side handle: kernels need its device address, which differs per GPU.
    // Resolve it once per device, with that device current (this is the set-up the first call performs).
    static std::mutex mu;
    static float* dev_ptr[64] = {};
    int dev = 0;
    if (int32_t s = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return s;
    MFT_CHECK_ARG(dev >= 0 && dev < 64, "mft_attn_bwd_noalloc: device index out of range");
    float* delta = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!dev_ptr[dev]) {
            void* p = nullptr;
            if (int32_t s = check_cuda(cudaGetSymbolAddress(&p, g_attn_noalloc_delta), "cudaGetSymbolAddress(attention scratch)")) return s;
            dev_ptr[dev] = static_cast<float*>(p);
        }
        delta = dev_ptr[dev];
    }
    // Every row the kernels read is first overwritten by the delta kernel of this call, so nothing needs clearing.
    return mft_attn_bwd(q, sq, k, sk, v, sv, o, so, d_o, sdo, lse, dq, dk, dv, delta, nullptr, batch, seq, n_heads, n_kv, hd, scale,
                        window, stream);
}
