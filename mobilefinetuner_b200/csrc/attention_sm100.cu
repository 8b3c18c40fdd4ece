// Causal / sliding-window GQA attention on the 5th-generation tensor cores (tcgen05) for head_dim 64, 128 and 256
// (the kernels are templates over the head size; the comments quote the sizes of head_dim 256).
//
// Forward: one CTA per (128 queries, head, batch).  Scores and the output accumulator live in tensor memory:
//     S = Q K^T      128 x 64 per key tile, two buffers (128 columns)
//     O += P V       128 x 256 (256 columns)
//     P              128 x 64 bf16 per key tile, two buffers (64 columns): the A operand of P V
// Warp 0 streams K and V tiles with TMA (128-byte swizzle; K two stages, V three: a V tile is held until its
// P V product is done), warp 1's one thread issues S, warp 10's one thread issues P V, warps 2..9 are the
// softmax: two threads share a query row (one tensor-memory lane, 32 of the tile's 64 keys each; they exchange
// their maxima through shared memory), apply the mask as an index predicate, exponentiate against a running
// reference maximum and store the bf16 probabilities back into tensor memory (tcgen05.st), from where the
// P V MMA reads them as its A operand (no shared-memory tile, no proxy fence on the softmax path).
// V is consumed as it lies in memory ([key][d], "MN-major" B operand), so nothing is transposed.
// The reference maximum is only raised (and O rescaled in tensor memory) when a row's maximum grew by more
// than 2^8 since the last rescale, which keeps the exponentials below 256 and makes rescales rare.
// Every mbarrier wait is bounded; a wait that runs out sets the library status word and the CTA leaves.
#include <cuda.h>

#include <cstdlib>

#include "attention.h"
#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

using namespace ptx;

namespace {

constexpr float LOG2E = 1.4426950408889634f;
constexpr int BM = 128, BN = 64;
constexpr int THREADS = 352;   // TMA warp, S-issuing warp, 8 softmax warps, P V-issuing warp
constexpr int FWD_VST = 3;                     // V stages (a V tile is held until its P V product is done; K only for S)
constexpr float RESCALE_GAP = 8.0f;            // log2 units
// Sizes that depend on the head size.  Rows of Q / K / V tiles are cut into CH boxes of 64 columns (128-byte rows).
template <int HD>
struct Dim {
    static_assert(HD == 64 || HD == 128 || HD == 256, "head_dim");
    static constexpr int CH = HD / 64;
    static constexpr int Q_BYTES = BM * HD * 2;            // CH boxes of [128 rows x 64 columns]
    static constexpr int KV_BYTES = BN * HD * 2;           // CH boxes of [64 rows x 64 columns]
    static constexpr int FWD_SMEM = Q_BYTES + (2 + FWD_VST) * KV_BYTES + 192 + 2 * 2 * BM * 4;   // head_dim 256: 231,616 of 232,448 bytes
    // forward tensor-memory columns: S buffers at 0 / 64, O at 128 .. 128 + HD, then the bf16 probabilities (the A operand
    // of P V: 32 columns = 64 keys per buffer)
    static constexpr int S_COL = 0, O_COL = 128, P_COL = 128 + HD;
    static constexpr int FWD_TMEM = HD == 64 ? 256 : 512;  // allocation (a power of two >= P_COL + 64)
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// A operand from tensor memory (lane = row, two bf16 of consecutive k per 32-bit column), B from shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}

// B operand stored [k][n] with n contiguous (128-byte swizzled boxes of 64 n-columns, `chunk_bytes` apart):
// leading byte offset = distance between 64-column chunks, stride byte offset = 1024 (8 k-rows).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t chunk_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((chunk_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
constexpr uint32_t IDESC_B_MN = 1u << 16;      // instruction-descriptor bit: B operand is MN-major

struct FwdParams {
    int seq, n_heads, rep, window;
    float scale;
    __nv_bfloat16* out;
    long long so_b, so_s, so_h;
    float* lse;
    int32_t* status;
    int q_col0_stride, kv_col0_stride;         // column of head h in the q / kv tensor maps = h * stride
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ bool visible(int i, int j, int window) { return j <= i && (window <= 0 || i - j < window); }

// head_dim 64 needs 58 KB of shared memory and 256 tensor-memory columns per CTA: two CTAs share an SM and cover each
// other's barrier / tensor-memory latencies (one tile's chain of S -> softmax -> P -> P V is several times longer than its
// MMAs)
template <int HD>
__global__ void __launch_bounds__(THREADS, HD == 64 ? 2 : 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
    dep_trigger();
    // The swizzled tiles need 1024-byte alignment and the tiles fill the SM's shared memory to within 1 KB, so
    // there is no room for alignment slack: the dynamic segment is declared aligned and checked below.
    constexpr int CH = Dim<HD>::CH, Q_BYTES = Dim<HD>::Q_BYTES, KV_BYTES = Dim<HD>::KV_BYTES;
    constexpr int S_COL = Dim<HD>::S_COL, O_COL = Dim<HD>::O_COL, P_COL = Dim<HD>::P_COL;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = smem_raw;
    uint8_t* q_smem = base;
    uint8_t* k_smem = q_smem + Q_BYTES;            // 2 stages
    uint8_t* v_smem = k_smem + 2 * KV_BYTES;       // FWD_VST stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + FWD_VST * KV_BYTES);
    uint64_t* q_full = bars;            // [1]
    uint64_t* k_full = bars + 1;        // [2]
    uint64_t* v_full = bars + 3;        // [3]
    uint64_t* k_empty = bars + 6;       // [2]
    uint64_t* v_empty = bars + 8;       // [3]
    uint64_t* s_full = bars + 11;       // [2]
    uint64_t* s_free = bars + 13;       // [2]  256 arrivals
    uint64_t* p_full = bars + 15;       // [2]  256 arrivals
    uint64_t* p_free = bars + 17;       // [2]
    uint64_t* o_done = bars + 19;       // [2]  P V product t completes o_done[t & 1] (two barriers, so that a waiter
                                        //      one product behind cannot mistake an older phase for the one it needs)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* mx_smem = reinterpret_cast<float*>(bars + 24);   // [2 buffers][2 halves][128] row maxima, later row sums
    float* l_smem = mx_smem;
    if ((smem_u32(smem_raw) & 1023u) != 0) {               // uniform: nothing has been allocated or armed yet
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, MFT_ERR_INVALID_ARG);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;     // longest rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.rep;
    const int i0 = qb * BM;
    const int jb_hi = (i0 + BM - 1) / BN;
    const int jb_lo = p.window > 0 ? max(0, i0 - p.window + 1) / BN : 0;
    const int n_tiles = jb_hi - jb_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 256); mbar_init(&p_full[s], 256); mbar_init(&p_free[s], 1);
        }
        for (int s = 0; s < FWD_VST; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        mbar_init(&o_done[0], 1); mbar_init(&o_done[1], 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, Dim<HD>::FWD_TMEM); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    dep_wait();     // set-up above overlapped the previous kernel's tail; its results are needed from here on

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            const int qx = h * p.q_col0_stride, kx = kvh * p.kv_col0_stride;
            mbar_arrive_expect_tx(q_full, Q_BYTES);
            for (int c = 0; c < CH; ++c) tma_load_2d(q_smem + c * (BM * 128), &map_q, q_full, qx + c * 64, b * p.seq + i0);
            int vs = 0;
            uint32_t vph = 0;                           // V stage of tile t and its phase parity
            for (int t = 0; t < n_tiles; ++t) {
                const int st = t & 1;
                const uint32_t ph = (t >> 1) & 1;
                const int row = b * p.seq + (jb_lo + t) * BN;
                if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&k_full[st], KV_BYTES);
                for (int c = 0; c < CH; ++c) tma_load_2d(k_smem + st * KV_BYTES + c * (BN * 128), &map_k, &k_full[st], kx + c * 64, row);
                if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&v_full[vs], KV_BYTES);
                for (int c = 0; c < CH; ++c) tma_load_2d(v_smem + vs * KV_BYTES + c * (BN * 128), &map_v, &v_full[vs], kx + c * 64, row);
                if (++vs == FWD_VST) { vs = 0; vph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer 1: S = Q K^T
        // (The tensor pipe takes MMAs from a thread only about as fast as that thread issues them: every wait,
        // fence and commit between two MMAs is exposed when the MMAs are short.  Two issuing threads overlap
        // one product's bookkeeping with the other product's MMAs.)
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16_f32(BM, BN);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            const uint64_t qd = smem_desc_sw128(smem_u32(q_smem));
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int st = t & 1;
                const uint32_t ph = (t >> 1) & 1;
                if (!mbar_wait(&k_full[st], ph, abort_flag) || !mbar_wait(&s_free[st], ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t kd = smem_desc_sw128(smem_u32(k_smem + st * KV_BYTES));
                const uint32_t tmem_s = tmem_base + S_COL + st * BN;
#pragma unroll
                for (int c = 0; c < CH; ++c)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_bf16(tmem_s, qd + (uint64_t)(c * (BM * 128 / 16) + 2 * j), kd + (uint64_t)(c * (BN * 128 / 16) + 2 * j), idesc_s,
                                  (c | j) != 0 ? 1u : 0u);
                umma_commit(&k_empty[st]);
                umma_commit(&s_full[st]);
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------ MMA issuer 2: O += P V
        if (lane == 0) {
            constexpr uint32_t idesc_o = idesc_bf16_f32(BM, HD) | IDESC_B_MN;
            bool ok = true;
            int vs = 0;
            uint32_t vph = 0;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int st = t & 1;
                const uint32_t ph = (t >> 1) & 1;
                if (!mbar_wait(&v_full[vs], vph, abort_flag) || !mbar_wait(&p_full[st], ph, abort_flag)) { ok = false; break; }
                tc_fence_after();
                // A = the bf16 probabilities in tensor memory (8 columns per 16 keys), B = V as it lies in memory
                const uint32_t pa = tmem_base + P_COL + st * 32;
                const uint64_t vd = smem_desc_mn_sw128(smem_u32(v_smem + vs * KV_BYTES), BN * 128);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    umma_bf16_ts(tmem_base + O_COL, pa + 8 * j, vd + (uint64_t)(j * (2048 / 16)), idesc_o, (t | j) != 0 ? 1u : 0u);
                umma_commit(&v_empty[vs]);
                umma_commit(&p_free[st]);
                umma_commit(&o_done[st]);
                if (++vs == FWD_VST) { vs = 0; vph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------ softmax (warps 2..9): two threads per query row (32 keys each)
        const int q4 = warp & 3;                       // tensor-memory lane quarter of this warp
        const int half = (warp - 2) >> 2;              // which 32 of the tile's 64 keys
        const int r = q4 * 32 + lane;                  // row within the tile
        const int i = i0 + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        float m_used = -INFINITY, l = 0.f;             // both threads of a row keep identical m_used; l is per half
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int st = t & 1;
            const uint32_t ph = (t >> 1) & 1;
            const int j0 = (jb_lo + t) * BN + half * 32;
            if (!mbar_wait(&s_full[st], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[32];
            tmem_ld_32x32(lane_addr + S_COL + st * BN + half * 32, sr);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&s_free[st]);                  // the scores are in registers: the buffer may be overwritten
            const bool need_mask = (j0 + 31 > i0) || (p.window > 0 && j0 < i0 + BM - p.window);
            if (need_mask) {
#pragma unroll
                for (int x = 0; x < 32; ++x)
                    if (!visible(i, j0 + x, p.window)) sr[x] = 0xff800000u;   // -inf
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) m4[e] = fmaxf(m4[e], __uint_as_float(sr[x + e]));
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2;      // scale > 0
            // the row maximum over both halves
            mx_smem[(st * 2 + half) * BM + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q4) : "memory");
            mx = fmaxf(mx, mx_smem[(st * 2 + (half ^ 1)) * BM + r]);
            // raise the reference maximum only when it is far behind; O and l are rescaled with it
            const bool first = m_used == -INFINITY;
            const bool need = !first && mx > m_used + RESCALE_GAP;
            if (__any_sync(0xffffffffu, need)) {
                // the previous P V product must have landed before O is modified (none is in flight after it:
                // the next one waits for the probabilities written below)
                if (!mbar_wait(&o_done[(t - 1) & 1], (uint32_t)(((t - 1) >> 1) & 1), abort_flag)) { ok = false; break; }
                tc_fence_after();
                const float f = need ? ex2(m_used - mx) : 1.0f;
#pragma unroll 1
                for (int c = 0; c < HD / 2; c += 32) {
                    uint32_t o[32];
                    tmem_ld_32x32(lane_addr + O_COL + half * (HD / 2) + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
                    tmem_st_32x32(lane_addr + O_COL + half * (HD / 2) + c, o);
                }
                tmem_st_wait();
                tc_fence_before();
                l *= f;
                if (need) m_used = mx;
            }
            if (first && mx > -INFINITY) m_used = mx;  // nothing accumulated yet for this row: no rescale needed
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[16];
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
                float e4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    e4[e] = ex2(fmaf(__uint_as_float(sr[x + e]), sl2, neg_m));      // -inf -> 0
                    ps[e] += e4[e];
                }
                const __nv_bfloat162 w0 = __floats2bfloat162_rn(e4[0], e4[1]), w1 = __floats2bfloat162_rn(e4[2], e4[3]);
                pk[x >> 1] = *reinterpret_cast<const uint32_t*>(&w0);
                pk[(x >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&w1);
            }
            l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            if (!mbar_wait(&p_free[st], ph ^ 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            tmem_st_32x16(lane_addr + P_COL + st * 32 + half * 16, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[st]);
        }
        // ---- epilogue: O / l -> bf16 (each thread its half of the row), row log-sum-exp
        const int lb = n_tiles & 1;                    // the exchange buffer the last tile did not use
        l_smem[(lb * 2 + half) * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + q4) : "memory");
        l += l_smem[(lb * 2 + (half ^ 1)) * BM + r];
        if (ok && mbar_wait(&o_done[(n_tiles - 1) & 1], (uint32_t)(((n_tiles - 1) >> 1) & 1), abort_flag)) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* orow = p.out + (long long)b * p.so_b + (long long)i * p.so_s + (long long)h * p.so_h + half * (HD / 2);
#pragma unroll 1
            for (int c = 0; c < HD / 2; c += 32) {
                uint32_t o[32];
                tmem_ld_32x32(lane_addr + O_COL + half * (HD / 2) + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 32; x += 8) {
                    float t8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) t8[e] = __uint_as_float(o[x + e]) * inv;
                    store8(orow + c + x, t8);
                }
            }
            if (half == 0) p.lse[((long long)b * p.n_heads + h) * p.seq + i] = (m_used + log2f(l)) / LOG2E;
        }
    }

    // ------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, MFT_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Dim<HD>::FWD_TMEM);
    }
}

// ---------------------------------------------------------------- backward: dQ
// One CTA per (128 queries, head, batch).  Q and dO stay in shared memory; K streams in 32-key tiles through
// four stages (held until the tile's dQ product), V through two.  Per tile: S = Q K^T and dP = dO V^T into tensor
// memory, the element-wise threads form dS = P (dP - delta) with P = exp2(S scale log2e - lse log2e) and store it
// as bf16 back into tensor memory, and dQ += dS K accumulates in tensor memory (dS read as the A operand from
// tensor memory, K consumed MN-major).  The element-wise work has no state across tiles, so two groups of 256
// threads (two threads per query row each) take alternate tiles and overlap each other's latency; group g owns
// S/dP buffer g and 16 tensor-memory columns for its dS.
constexpr int DQ_BN = 32;
constexpr int DQ_KST = 4, DQ_VST = 2;              // K / V stages (K is held until the tile's dQ product, V only for dP)
// Threads: TMA warp, S issuer, GROUPS x 8 element-wise warps, dP issuer, dQ issuer.  With two groups, group g works on
// the tiles t = g, g + 2, ... (tensor-memory buffer g); head_dim 64 runs ONE group that takes every tile (buffer t & 1):
// 384 threads, 58 KB of shared memory and 256 tensor-memory columns per CTA let two CTAs share an SM, and the second
// CTA's independent chain covers the first one's barrier / tensor-memory latencies.
constexpr int DQ_S_COL = 0, DQ_DP_COL = 64, DQ_ACC_COL = 128;
template <int HD>
struct DqDim {
    static constexpr int KV_BYTES = DQ_BN * HD * 2;    // CH chunks of [32 rows x 64 columns]
    static constexpr int SMEM = 2 * Dim<HD>::Q_BYTES + (DQ_KST + DQ_VST) * KV_BYTES + 256 + 4 * BM * 4;
    static constexpr int DS_COL = 128 + HD;            // dS as the A operand of the dQ product: 16 columns (32 keys as bf16 pairs) per group
    static constexpr int TMEM = HD == 64 ? 256 : 512;
    static constexpr int GROUPS = HD == 64 ? 1 : 2;
    static constexpr int THREADS = 64 + GROUPS * 256 + 64;
    static constexpr int W_DP = 2 + 8 * GROUPS, W_DQ = 3 + 8 * GROUPS;   // warps of the dP and dQ issuers
};


struct BwdParams {
    int seq, n_heads, n_kv, rep, window;
    float scale;
    const float* lse;
    const float* delta;
    __nv_bfloat16* dq;
    long long sq_b, sq_s, sq_h;
    float* dkv_acc;
    int32_t* status;
    int q_col0_stride, do_col0_stride, k_col0_stride, v_col0_stride;
    // dQ kernel only: when o != nullptr the kernel first forms delta[row] = sum_d O * dO for its rows and stores it
    const __nv_bfloat16 *o, *d_o;
    long long so_b, so_s, so_h, sdo_b, sdo_s, sdo_h;
    float* delta_out;
};

template <int HD>
__global__ void __launch_bounds__(DqDim<HD>::THREADS, DqDim<HD>::GROUPS == 1 ? 2 : 1)
attn_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                  const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const BwdParams p) {
    dep_trigger();
    constexpr int CH = Dim<HD>::CH, Q_BYTES = Dim<HD>::Q_BYTES, DQ_KV_BYTES = DqDim<HD>::KV_BYTES, DQ_DS_COL = DqDim<HD>::DS_COL;
    constexpr int GROUPS = DqDim<HD>::GROUPS, W_DP = DqDim<HD>::W_DP, W_DQ = DqDim<HD>::W_DQ;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* q_smem = smem_raw;
    uint8_t* do_smem = q_smem + Q_BYTES;
    uint8_t* k_smem = do_smem + Q_BYTES;                   // DQ_KST stages
    uint8_t* v_smem = k_smem + DQ_KST * DQ_KV_BYTES;       // DQ_VST stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + DQ_VST * DQ_KV_BYTES);
    uint64_t* qdo_full = bars;          // [1]
    uint64_t* k_full = bars + 1;        // [4]
    uint64_t* k_empty = bars + 5;       // [4]
    uint64_t* v_full = bars + 9;        // [2]
    uint64_t* v_empty = bars + 11;      // [2]
    uint64_t* sdp_full = bars + 13;     // [2]  per group; two arrivals (S and dP)
    uint64_t* sdp_free = bars + 15;     // [2]  256 arrivals
    uint64_t* ds_full = bars + 17;      // [2]  256 arrivals
    uint64_t* ds_free = bars + 19;      // [2]
    uint64_t* acc_done = bars + 21;     // [1]  completed once, by the last dQ product
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* delta_smem = reinterpret_cast<float*>(bars + 32);   // [4][128] partial rowsum(O * dO) of this CTA's queries
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, MFT_ERR_INVALID_ARG);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / p.rep;
    const int i0 = qb * BM;
    const int jb_hi = (i0 + BM - 1) / DQ_BN;
    const int jb_lo = p.window > 0 ? max(0, i0 - p.window + 1) / DQ_BN : 0;
    const int n_tiles = jb_hi - jb_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(qdo_full, 1);
        for (int s = 0; s < DQ_KST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&sdp_full[s], 2); mbar_init(&sdp_free[s], 256); mbar_init(&ds_full[s], 256); mbar_init(&ds_free[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, DqDim<HD>::TMEM); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    dep_wait();     // set-up above overlapped the previous kernel's tail; its results are needed from here on

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(qdo_full, 2 * Q_BYTES);
            for (int c = 0; c < CH; ++c) tma_load_2d(q_smem + c * (BM * 128), &map_q, qdo_full, h * p.q_col0_stride + c * 64, b * p.seq + i0);
            for (int c = 0; c < CH; ++c) tma_load_2d(do_smem + c * (BM * 128), &map_do, qdo_full, h * p.do_col0_stride + c * 64, b * p.seq + i0);
            for (int t = 0; t < n_tiles; ++t) {
                const int ks = t % DQ_KST, vs = t & 1;
                const uint32_t kph = (t / DQ_KST) & 1, vph = (t >> 1) & 1;
                const int row = b * p.seq + (jb_lo + t) * DQ_BN;
                if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&k_full[ks], DQ_KV_BYTES);
                for (int c = 0; c < CH; ++c) tma_load_2d(k_smem + ks * DQ_KV_BYTES + c * (DQ_BN * 128), &map_k, &k_full[ks], kvh * p.k_col0_stride + c * 64, row);
                if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&v_full[vs], DQ_KV_BYTES);
                for (int c = 0; c < CH; ++c) tma_load_2d(v_smem + vs * DQ_KV_BYTES + c * (DQ_BN * 128), &map_v, &v_full[vs], kvh * p.v_col0_stride + c * 64, row);
            }
        }
    } else if (warp == 1 || warp == W_DP) {
        // ------------------------------------------------ MMA issuers 1 and 2: S = Q K^T (warp 1), dP = dO V^T (warp W_DP)
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16_f32(BM, DQ_BN);
            const bool is_s = warp == 1;
            bool ok = mbar_wait(qdo_full, 0, abort_flag);
            const uint64_t ad = smem_desc_sw128(smem_u32(is_s ? q_smem : do_smem));
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int g = t & 1, ks = t % DQ_KST;
                const uint32_t gph = (t >> 1) & 1, kph = (t / DQ_KST) & 1;
                if (is_s ? !mbar_wait(&k_full[ks], kph, abort_flag) : !mbar_wait(&v_full[g], gph, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&sdp_free[g], gph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t bd = smem_desc_sw128(smem_u32(is_s ? k_smem + ks * DQ_KV_BYTES : v_smem + g * DQ_KV_BYTES));
                const uint32_t tmem_d = tmem_base + (is_s ? DQ_S_COL : DQ_DP_COL) + g * DQ_BN;
#pragma unroll
                for (int c = 0; c < CH; ++c)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_bf16(tmem_d, ad + (uint64_t)(c * (BM * 128 / 16) + 2 * j), bd + (uint64_t)(c * (DQ_BN * 128 / 16) + 2 * j), idesc_s,
                                  (c | j) != 0 ? 1u : 0u);
                if (!is_s) umma_commit(&v_empty[g]);
                umma_commit(&sdp_full[g]);            // two arrivals complete it: S and dP
            }
        }
    } else if (warp == W_DQ) {
        // ------------------------------------------------ MMA issuer 3: dQ += dS K
        if (lane == 0) {
            constexpr uint32_t idesc_acc = idesc_bf16_f32(BM, HD) | IDESC_B_MN;
            bool ok = true;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int g = t & 1, ks = t % DQ_KST;
                const uint32_t gph = (t >> 1) & 1;
                if (!mbar_wait(&ds_full[g], gph, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t kd = smem_desc_mn_sw128(smem_u32(k_smem + ks * DQ_KV_BYTES), DQ_BN * 128);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    umma_bf16_ts(tmem_base + DQ_ACC_COL, tmem_base + DQ_DS_COL + g * 16 + 8 * j, kd + (uint64_t)(j * (2048 / 16)), idesc_acc, (t | j) != 0 ? 1u : 0u);
                umma_commit(&k_empty[ks]);
                umma_commit(&ds_free[g]);
                if (t == n_tiles - 1) umma_commit(acc_done);
            }
        }
    } else {
        const int g0 = (warp - 2) >> 3;                // element-wise group: tiles t = g0, g0 + GROUPS, ...
        const int q4 = warp & 3;
        const int half = ((warp - 2) >> 2) & 1;        // which 16 of the tile's 32 keys
        const int r = q4 * 32 + lane;
        const int i = i0 + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        const long long sidx = ((long long)b * p.n_heads + h) * p.seq + i;
        const float neg_lse2 = -p.lse[sidx] * LOG2E;
        float dlt;
        if (HD == 256 && p.o != nullptr) {
            // delta = rowsum(O * dO): the four element-wise threads of a row (2 groups x 2 halves) take 64 columns
            // each, the partial sums meet in shared memory; thread (group 0, half 0) stores the row's delta for the
            // dK/dV kernel
            {
                const int part = g0 * 2 + half;
                const __nv_bfloat16* orow = p.o + (long long)b * p.so_b + (long long)i * p.so_s + (long long)h * p.so_h + part * 64;
                const __nv_bfloat16* drow = p.d_o + (long long)b * p.sdo_b + (long long)i * p.sdo_s + (long long)h * p.sdo_h + part * 64;
                float a8[8][8], c8[8][8];
#pragma unroll
                for (int d = 0; d < 8; ++d) { load8(orow + d * 8, a8[d]); load8(drow + d * 8, c8[d]); }
                float acc = 0.f;
#pragma unroll
                for (int d = 0; d < 8; ++d)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc = fmaf(a8[d][e], c8[d][e], acc);
                delta_smem[part * BM + r] = acc;
            }
            asm volatile("bar.sync 1, 512;" ::: "memory");     // the 16 element-wise warps
            const float dsum = (delta_smem[r] + delta_smem[BM + r]) + (delta_smem[2 * BM + r] + delta_smem[3 * BM + r]);
            if (g0 == 0 && half == 0) p.delta_out[sidx] = dsum;
            dlt = dsum;
        } else {
            dlt = p.delta[sidx];
        }
        bool ok = true;
        for (int t = g0; t < n_tiles && ok; t += GROUPS) {
            const int g = t & 1;                       // tensor-memory buffer of the tile
            const uint32_t ph = (t >> 1) & 1;
            const int j0 = (jb_lo + t) * DQ_BN + half * 16;
            if (!mbar_wait(&sdp_full[g], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[16], dr[16];
            tmem_ld_32x16(lane_addr + DQ_S_COL + g * DQ_BN + half * 16, sr);
            tmem_ld_32x16(lane_addr + DQ_DP_COL + g * DQ_BN + half * 16, dr);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&sdp_free[g]);
            const bool need_mask = (j0 + 15 > i0) || (p.window > 0 && j0 < i0 + BM - p.window);
            uint32_t pk[8];
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
                float d2[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float pv = ex2(fmaf(__uint_as_float(sr[x + e]), sl2, neg_lse2));
                    if (need_mask && !visible(i, j0 + x + e, p.window)) pv = 0.f;
                    d2[e] = pv * (__uint_as_float(dr[x + e]) - dlt);
                }
                const __nv_bfloat162 w = __floats2bfloat162_rn(d2[0], d2[1]);
                pk[x >> 1] = *reinterpret_cast<const uint32_t*>(&w);
            }
            if (!mbar_wait(&ds_free[g], ph ^ 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            tmem_st_32x8(lane_addr + DQ_DS_COL + g * 16 + half * 8, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&ds_full[g]);
        }
        if (g0 == 0 && ok && mbar_wait(acc_done, 0, abort_flag)) {
            tc_fence_after();
            __nv_bfloat16* row = p.dq + (long long)b * p.sq_b + (long long)i * p.sq_s + (long long)h * p.sq_h + half * (HD / 2);
#pragma unroll 1
            for (int c = 0; c < HD / 2; c += 32) {
                uint32_t o[32];
                tmem_ld_32x32(lane_addr + DQ_ACC_COL + half * (HD / 2) + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 32; x += 8) {
                    float t8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) t8[e] = __uint_as_float(o[x + e]) * p.scale;
                    store8(row + c + x, t8);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, MFT_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, DqDim<HD>::TMEM);
    }
}

// ---------------------------------------------------------------- backward: dK, dV
// One CTA per (128 keys, query head, half of head_dim, batch): dK and dV for 128 keys x 256 columns would fill
// the whole tensor memory, so each CTA accumulates 128 of the 256 columns (both halves recompute S and dP).
// K and V stay in shared memory; Q, dO and the per-query log-sum-exp / delta stream in 32-query tiles through
// three stages (a stage is held until the tile's dV / dK products are done, and the next load into it takes
// longer than one tile's MMAs: with two stages the tensor pipe waited for it).  Per tile: S^T = K Q^T and
// dP^T = V dO^T (128 keys x 32 queries) into tensor memory, element-wise group t & 1 forms P^T and dS^T and stores
// them as bf16 back into tensor memory (32 columns per group), and dV += P^T dO, dK += dS^T Q accumulate in tensor
// memory with P^T / dS^T read as A operands from tensor memory and dO / Q consumed MN-major from the stage.
// The result is added into the caller's f32 [2][batch, seq, n_kv, 256] scratch (query heads of a KV group and
// the two halves write disjoint columns or add).
constexpr int KV_BQ = 32;                              // queries per tile
constexpr int KV_STATS_BYTES = 2 * KV_BQ * 4;          // lse, delta of the tile's queries
constexpr int KV_STAGES = 3;                           // Q / dO stages: the load of tile t+2 must not wait for the MMAs of tile t
// Threads: TMA warp, S^T issuer, GROUPS x 8 element-wise warps, dP^T issuer, dV/dK issuer.  head_dim 64 runs one group
// and keeps P^T / dS^T IN PLACE (each element-wise thread writes its 16 bf16 probabilities over the first 8 of the 16
// S^T columns it has just read, dS^T likewise over dP^T): 256 tensor-memory columns, 384 threads and 57 KB of shared
// memory per CTA, so that two CTAs share an SM.  The S^T / dP^T buffers are then free again only when the tile's
// dV / dK products have read them.
constexpr int KV_S_COL = 0, KV_DP_COL = 64, KV_DK_COL = 128;
template <int HD>
struct KvDim {
    static constexpr int ACC = HD == 256 ? 128 : HD;   // head_dim columns one CTA accumulates (head_dim 256: two CTAs per head)
    static constexpr int NPART = HD / ACC;
    static constexpr int Q_BYTES = KV_BQ * HD * 2;     // CH chunks of [32 rows x 64 columns]
    static constexpr int SMEM = 2 * Dim<HD>::Q_BYTES + KV_STAGES * 2 * Q_BYTES + KV_STAGES * KV_STATS_BYTES + 256;
    static constexpr int DV_COL = KV_DK_COL + ACC;
    static constexpr int PDS_COL = KV_DK_COL + 2 * ACC;   // per group 32 columns: P^T (16: 32 queries as bf16 pairs) | dS^T (16)
    static constexpr bool INPLACE = HD == 64;
    static constexpr int TMEM = INPLACE ? 256 : 512;
    static constexpr int GROUPS = HD == 64 ? 1 : 2;
    static constexpr int THREADS = 64 + GROUPS * 256 + 64;
    static constexpr int W_DP = 2 + 8 * GROUPS, W_ACC = 3 + 8 * GROUPS;   // warps of the dP^T and dV/dK issuers
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(smem_u32(smem_dst)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

template <int HD>
__global__ void __launch_bounds__(KvDim<HD>::THREADS, KvDim<HD>::GROUPS == 1 ? 2 : 1)
attn_dkv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const BwdParams p) {
    dep_trigger();
    constexpr int CH = Dim<HD>::CH, Q_BYTES = Dim<HD>::Q_BYTES, KV_Q_BYTES = KvDim<HD>::Q_BYTES, ACC = KvDim<HD>::ACC, NPART = KvDim<HD>::NPART;
    constexpr int KV_DV_COL = KvDim<HD>::DV_COL, KV_PDS_COL = KvDim<HD>::PDS_COL;
    constexpr bool INPLACE = KvDim<HD>::INPLACE;
    constexpr int GROUPS = KvDim<HD>::GROUPS, W_DP = KvDim<HD>::W_DP, W_ACC = KvDim<HD>::W_ACC;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* k_smem = smem_raw;                            // [128 keys x 256], 4 chunks
    uint8_t* v_smem = k_smem + Q_BYTES;
    uint8_t* q_smem = v_smem + Q_BYTES;                    // KV_STAGES stages
    uint8_t* do_smem = q_smem + KV_STAGES * KV_Q_BYTES;    // KV_STAGES stages
    float* stats = reinterpret_cast<float*>(do_smem + KV_STAGES * KV_Q_BYTES);   // [stage][lse 32 | delta 32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stats) + KV_STAGES * KV_STATS_BYTES);
    uint64_t* kv_full = bars;           // [1]
    uint64_t* qdo_full = bars + 1;      // [3]
    uint64_t* qdo_empty = bars + 4;     // [3]
    uint64_t* sdp_full = bars + 7;      // [2]  two arrivals (S^T and dP^T)
    uint64_t* sdp_free = bars + 9;      // [2]  256 arrivals
    uint64_t* pds_full = bars + 11;     // [2]  256 arrivals
    uint64_t* pds_free = bars + 13;     // [2]
    uint64_t* acc_done = bars + 15;     // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, MFT_ERR_INVALID_ARG);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int jb = blockIdx.x, b = blockIdx.z;
    const int h = blockIdx.y / NPART, hh = blockIdx.y % NPART;    // query head, part of head_dim
    const int kvh = h / p.rep;
    const int j0 = jb * BM;
    // queries that can see keys j0 .. j0+127: i >= j0 and i - j < window
    const int i_max = p.window > 0 ? min(p.seq - 1, j0 + BM - 1 + p.window - 1) : p.seq - 1;
    const int qs_lo = j0 / KV_BQ, qs_hi = i_max / KV_BQ;
    const int n_tiles = qs_hi - qs_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sdp_full[s], 2); mbar_init(&sdp_free[s], 256); mbar_init(&pds_full[s], 256); mbar_init(&pds_free[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, KvDim<HD>::TMEM); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    dep_wait();     // set-up above overlapped the previous kernel's tail; its results are needed from here on

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(kv_full, 2 * Q_BYTES);
            for (int c = 0; c < CH; ++c) tma_load_2d(k_smem + c * (BM * 128), &map_k, kv_full, kvh * p.k_col0_stride + c * 64, b * p.seq + j0);
            for (int c = 0; c < CH; ++c) tma_load_2d(v_smem + c * (BM * 128), &map_v, kv_full, kvh * p.v_col0_stride + c * 64, b * p.seq + j0);
            const long long srow = ((long long)b * p.n_heads + h) * p.seq;
            int st = 0;
            uint32_t sph = 0;                           // stage of tile t and its phase parity (t / KV_STAGES) & 1
            for (int t = 0; t < n_tiles; ++t) {
                const int i0 = (qs_lo + t) * KV_BQ;
                if (!mbar_wait(&qdo_empty[st], sph ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&qdo_full[st], 2 * KV_Q_BYTES + KV_STATS_BYTES);
                for (int c = 0; c < CH; ++c) tma_load_2d(q_smem + st * KV_Q_BYTES + c * (KV_BQ * 128), &map_q, &qdo_full[st], h * p.q_col0_stride + c * 64, b * p.seq + i0);
                for (int c = 0; c < CH; ++c) tma_load_2d(do_smem + st * KV_Q_BYTES + c * (KV_BQ * 128), &map_do, &qdo_full[st], h * p.do_col0_stride + c * 64, b * p.seq + i0);
                bulk_load_1d(stats + st * 2 * KV_BQ, p.lse + srow + i0, KV_BQ * 4, &qdo_full[st]);
                bulk_load_1d(stats + st * 2 * KV_BQ + KV_BQ, p.delta + srow + i0, KV_BQ * 4, &qdo_full[st]);
                if (++st == KV_STAGES) { st = 0; sph ^= 1; }
            }
        }
    } else if (warp == 1 || warp == W_DP) {
        // ------------------------------------------------ MMA issuers 1 and 2: S^T = K Q^T (warp 1), dP^T = V dO^T (warp W_DP)
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16_f32(BM, KV_BQ);
            const bool is_s = warp == 1;
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            const uint64_t ad = smem_desc_sw128(smem_u32(is_s ? k_smem : v_smem));
            int st = 0;
            uint32_t sph = 0;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int g = t & 1;
                const uint32_t ph = (t >> 1) & 1;
                // in place: the buffer also holds P^T / dS^T of tile t - 2 until that tile's dV / dK products are done
                if (!mbar_wait(&qdo_full[st], sph, abort_flag) || !mbar_wait(INPLACE ? &pds_free[g] : &sdp_free[g], ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t bd = smem_desc_sw128(smem_u32((is_s ? q_smem : do_smem) + st * KV_Q_BYTES));
                const uint32_t tmem_d = tmem_base + (is_s ? KV_S_COL : KV_DP_COL) + g * KV_BQ;
#pragma unroll
                for (int c = 0; c < CH; ++c)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_bf16(tmem_d, ad + (uint64_t)(c * (BM * 128 / 16) + 2 * j), bd + (uint64_t)(c * (KV_BQ * 128 / 16) + 2 * j), idesc_s,
                                  (c | j) != 0 ? 1u : 0u);
                umma_commit(&sdp_full[g]);
                if (++st == KV_STAGES) { st = 0; sph ^= 1; }
            }
        }
    } else if (warp == W_ACC) {
        // ------------------------------------------------ MMA issuer 3: dV += P^T dO, dK += dS^T Q (this CTA's 128 columns)
        if (lane == 0) {
            constexpr uint32_t idesc_acc = idesc_bf16_f32(BM, ACC) | IDESC_B_MN;
            bool ok = true;
            int st = 0;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int g = t & 1;
                const uint32_t ph = (t >> 1) & 1;
                if (!mbar_wait(&pds_full[g], ph, abort_flag)) { ok = false; break; }
                tc_fence_after();
                // A operands P^T / dS^T come from tensor memory (8 columns per 16 queries), B operands dO / Q MN-major from the stage
                // separate: P^T at pa + {0, 8}, dS^T at pa + 16 + {0, 8}.  In place: P^T in the S^T buffer at +{0, 16}
                // (the first 8 columns of each half's 16), dS^T in the dP^T buffer likewise
                const uint32_t pa = tmem_base + (INPLACE ? KV_S_COL + g * KV_BQ : KV_PDS_COL + g * 32);
                const uint32_t da = INPLACE ? tmem_base + KV_DP_COL + g * KV_BQ : pa + 16;
                constexpr int A_STEP = INPLACE ? 16 : 8;
                const uint64_t dod = smem_desc_mn_sw128(smem_u32(do_smem + st * KV_Q_BYTES + hh * (ACC / 64) * (KV_BQ * 128)), KV_BQ * 128);
                const uint64_t qd = smem_desc_mn_sw128(smem_u32(q_smem + st * KV_Q_BYTES + hh * (ACC / 64) * (KV_BQ * 128)), KV_BQ * 128);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    umma_bf16_ts(tmem_base + KV_DV_COL, pa + A_STEP * j, dod + (uint64_t)(j * (2048 / 16)), idesc_acc, (t | j) != 0 ? 1u : 0u);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    umma_bf16_ts(tmem_base + KV_DK_COL, da + A_STEP * j, qd + (uint64_t)(j * (2048 / 16)), idesc_acc, (t | j) != 0 ? 1u : 0u);
                umma_commit(&qdo_empty[st]);
                umma_commit(&pds_free[g]);
                if (t == n_tiles - 1) umma_commit(acc_done);
                if (++st == KV_STAGES) st = 0;
            }
        }
    } else {
        // ------------------------------------------------ element-wise groups (warps 2 .. 1 + 8 * GROUPS): key row per thread pair
        const int g0 = (warp - 2) >> 3;                // tiles t = g0, g0 + GROUPS, ...
        const int q4 = warp & 3;
        const int half = ((warp - 2) >> 2) & 1;        // which 16 of the tile's 32 queries
        const int r = q4 * 32 + lane;                  // key within the tile
        const int j = j0 + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        bool ok = true;
        for (int t = g0; t < n_tiles && ok; t += GROUPS) {
            const int g = t & 1;                       // tensor-memory buffer of the tile
            const uint32_t ph = (t >> 1) & 1;
            const int i0 = (qs_lo + t) * KV_BQ + half * 16;
            if (!mbar_wait(&sdp_full[g], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[16], dr[16];
            tmem_ld_32x16(lane_addr + KV_S_COL + g * KV_BQ + half * 16, sr);
            tmem_ld_32x16(lane_addr + KV_DP_COL + g * KV_BQ + half * 16, dr);
            tmem_ld_wait();
            tc_fence_before();
            if (!INPLACE) mbar_arrive(&sdp_free[g]);
            // lse / delta of the 16 queries (the stage's loads completed before S^T was issued)
            const float* st_l = stats + (t % KV_STAGES) * 2 * KV_BQ + half * 16;
            const float* st_d = st_l + KV_BQ;
            const bool need_mask = (i0 < j0 + BM - 1) || (p.window > 0 && i0 + 15 - j0 >= p.window);
            uint32_t pk[8], dk[8];
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
                float p2[2], d2[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float pv = ex2(fmaf(__uint_as_float(sr[x + e]), sl2, -st_l[x + e] * LOG2E));
                    if (need_mask && !visible(i0 + x + e, j, p.window)) pv = 0.f;
                    p2[e] = pv;
                    d2[e] = pv * (__uint_as_float(dr[x + e]) - st_d[x + e]);
                }
                const __nv_bfloat162 w0 = __floats2bfloat162_rn(p2[0], p2[1]), w1 = __floats2bfloat162_rn(d2[0], d2[1]);
                pk[x >> 1] = *reinterpret_cast<const uint32_t*>(&w0);
                dk[x >> 1] = *reinterpret_cast<const uint32_t*>(&w1);
            }
            if (INPLACE) {
                // over the first 8 of the 16 columns this thread has just read (nobody else touches them; the buffer
                // is this tile's until its dV / dK products complete pds_free, which the S^T / dP^T issuers wait for)
                tmem_st_32x8(lane_addr + KV_S_COL + g * KV_BQ + half * 16, pk);
                tmem_st_32x8(lane_addr + KV_DP_COL + g * KV_BQ + half * 16, dk);
            } else {
                if (!mbar_wait(&pds_free[g], ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                tmem_st_32x8(lane_addr + KV_PDS_COL + g * 32 + half * 8, pk);
                tmem_st_32x8(lane_addr + KV_PDS_COL + g * 32 + 16 + half * 8, dk);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&pds_full[g]);
        }
        // ---- epilogue (group 0): add this CTA's 128 columns of dK (scaled) and dV into the f32 scratch
        if (g0 == 0 && ok && mbar_wait(acc_done, 0, abort_flag)) {
            tc_fence_after();
            const long long half_elems = (long long)gridDim.z * p.seq * p.n_kv * HD;
            float* krow = p.dkv_acc + (((long long)b * p.seq + j) * p.n_kv + kvh) * HD + hh * ACC + half * (ACC / 2);
            float* vrow = krow + half_elems;
#pragma unroll 1
            for (int c = 0; c < ACC / 2; c += 32) {
                uint32_t o[32];
                tmem_ld_32x32(lane_addr + KV_DK_COL + half * (ACC / 2) + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 32; x += 4)
                    atomicAdd(reinterpret_cast<float4*>(krow + c + x), make_float4(__uint_as_float(o[x]) * p.scale, __uint_as_float(o[x + 1]) * p.scale,
                                                                                 __uint_as_float(o[x + 2]) * p.scale, __uint_as_float(o[x + 3]) * p.scale));
                tmem_ld_32x32(lane_addr + KV_DV_COL + half * (ACC / 2) + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int x = 0; x < 32; x += 4)
                    atomicAdd(reinterpret_cast<float4*>(vrow + c + x), make_float4(__uint_as_float(o[x]), __uint_as_float(o[x + 1]),
                                                                                 __uint_as_float(o[x + 2]), __uint_as_float(o[x + 3])));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, MFT_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, KvDim<HD>::TMEM);
    }
}

bool token_major(const mft_strides_t& s, int seq) { return s.stride_b == (int64_t)seq * s.stride_s; }

bool tc_shape_ok(int hd) { return hd == 64 || hd == 128 || hd == 256; }

template <int HD>
int32_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdParams& p, dim3 grid, cudaStream_t stream) {
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dim<HD>::FWD_SMEM), "attention smem attribute")) return s;
        configured = true;
    }
    launch_dep(attn_fwd_tc_kernel<HD>, dim3(grid), dim3(THREADS), (size_t)(Dim<HD>::FWD_SMEM), stream, mq, mk, mv, p);
    MFT_LAUNCH_CHECK("attn_fwd_tc");
    return MFT_OK;
}
template <int HD>
int32_t launch_dq(const CUtensorMap& mq, const CUtensorMap& md, const CUtensorMap& mk, const CUtensorMap& mv, const BwdParams& p, dim3 grid, cudaStream_t stream) {
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(attn_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqDim<HD>::SMEM), "attention smem attribute")) return s;
        configured = true;
    }
    launch_dep(attn_dq_tc_kernel<HD>, dim3(grid), dim3(DqDim<HD>::THREADS), (size_t)(DqDim<HD>::SMEM), stream, mq, md, mk, mv, p);
    MFT_LAUNCH_CHECK("attn_dq_tc");
    return MFT_OK;
}
template <int HD>
int32_t launch_dkv(const CUtensorMap& mq, const CUtensorMap& md, const CUtensorMap& mk, const CUtensorMap& mv, const BwdParams& p, int seq, int n_heads, int batch,
                   cudaStream_t stream) {
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(attn_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, KvDim<HD>::SMEM), "attention smem attribute")) return s;
        configured = true;
    }
    dim3 grid((unsigned)(seq / BM), (unsigned)(KvDim<HD>::NPART * n_heads), (unsigned)batch);
    launch_dep(attn_dkv_tc_kernel<HD>, dim3(grid), dim3(KvDim<HD>::THREADS), (size_t)(KvDim<HD>::SMEM), stream, mq, md, mk, mv, p);
    MFT_LAUNCH_CHECK("attn_dkv_tc");
    return MFT_OK;
}
#define HD_DISPATCH(hd, CALL64, CALL128, CALL256) ((hd) == 64 ? (CALL64) : (hd) == 128 ? (CALL128) : (CALL256))

}  // namespace

int32_t attn_fwd_sm100(const AttnParams& a, int hd, cudaStream_t stream) {
    static const int enabled = [] { const char* e = std::getenv("MFT_ATTN_TC"); return e ? std::atoi(e) : 1; }();
    if (!enabled || !tc_shape_ok(hd) || a.seq % BM != 0 || !device_status_word()) return MFT_ERR_UNSUPPORTED;
    // measured (batch 8, 14 / 2 heads of 64): at 256 tokens the mma.sync forward is faster (0.0205 against 0.0225 ms),
    // from 512 tokens on this kernel wins (0.039 against 0.041 ms, 2.3 x at 4096); MFT_ATTN_TC=2 forces it
    if (hd != 256 && a.seq < 512 && enabled < 2) return MFT_ERR_UNSUPPORTED;
    if (!token_major(a.sq, a.seq) || !token_major(a.sk, a.seq) || !token_major(a.sv, a.seq)) return MFT_ERR_UNSUPPORTED;
    if (a.sq.stride_h % 8 || a.sk.stride_h % 8 || a.sv.stride_h % 8 || a.so.stride_s % 8 || a.so.stride_h % 8 || a.so.stride_b % 8) return MFT_ERR_UNSUPPORTED;
    if ((int64_t)a.batch * a.seq >= (1ll << 31)) return MFT_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    const int64_t rows = (int64_t)a.batch * a.seq;
    if (make_tmap_bf16(&mq, a.q, rows, (int64_t)(a.n_heads - 1) * a.sq.stride_h + hd, a.sq.stride_s, BM) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mk, a.k, rows, (int64_t)(a.n_kv - 1) * a.sk.stride_h + hd, a.sk.stride_s, BN) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mv, a.v, rows, (int64_t)(a.n_kv - 1) * a.sv.stride_h + hd, a.sv.stride_s, BN) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (a.sk.stride_h != a.sv.stride_h) return MFT_ERR_UNSUPPORTED;
    FwdParams p{};
    p.seq = a.seq; p.n_heads = a.n_heads; p.rep = a.rep; p.window = a.window; p.scale = a.scale;
    p.out = a.out; p.so_b = a.so.stride_b; p.so_s = a.so.stride_s; p.so_h = a.so.stride_h; p.lse = a.lse;
    p.status = device_status_word();
    p.q_col0_stride = (int)a.sq.stride_h; p.kv_col0_stride = (int)a.sk.stride_h;
    dim3 grid((unsigned)(a.seq / BM), (unsigned)a.n_heads, (unsigned)a.batch);
    return HD_DISPATCH(hd, launch_fwd<64>(mq, mk, mv, p, grid, stream), launch_fwd<128>(mq, mk, mv, p, grid, stream), launch_fwd<256>(mq, mk, mv, p, grid, stream));
}

int32_t attn_dq_sm100(const AttnParams& a, int hd, bool compute_delta, cudaStream_t stream) {
    static const int enabled = [] { const char* e = std::getenv("MFT_ATTN_TC"); return e ? std::atoi(e) : 1; }();
    if (!enabled || !tc_shape_ok(hd) || a.seq % BM != 0 || !device_status_word()) return MFT_ERR_UNSUPPORTED;
    // the backward kernels win from 256 tokens on (0.064 against 0.073 ms at 256, 2.6 x at 4096); MFT_ATTN_TC=2 forces them
    if (hd != 256 && a.seq < 256 && enabled < 2) return MFT_ERR_UNSUPPORTED;
    if (compute_delta && hd != 256) return MFT_ERR_UNSUPPORTED;
    if (!token_major(a.sq, a.seq) || !token_major(a.sk, a.seq) || !token_major(a.sv, a.seq) || !token_major(a.sdo, a.seq)) return MFT_ERR_UNSUPPORTED;
    if (a.sq.stride_h % 8 || a.sk.stride_h % 8 || a.sv.stride_h % 8 || a.sdo.stride_h % 8) return MFT_ERR_UNSUPPORTED;
    if ((int64_t)a.batch * a.seq >= (1ll << 31)) return MFT_ERR_UNSUPPORTED;
    CUtensorMap mq, md, mk, mv;
    const int64_t rows = (int64_t)a.batch * a.seq;
    if (make_tmap_bf16(&mq, a.q, rows, (int64_t)(a.n_heads - 1) * a.sq.stride_h + hd, a.sq.stride_s, BM) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&md, a.d_o, rows, (int64_t)(a.n_heads - 1) * a.sdo.stride_h + hd, a.sdo.stride_s, BM) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mk, a.k, rows, (int64_t)(a.n_kv - 1) * a.sk.stride_h + hd, a.sk.stride_s, DQ_BN) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mv, a.v, rows, (int64_t)(a.n_kv - 1) * a.sv.stride_h + hd, a.sv.stride_s, DQ_BN) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    BwdParams p{};
    p.seq = a.seq; p.n_heads = a.n_heads; p.n_kv = a.n_kv; p.rep = a.rep; p.window = a.window; p.scale = a.scale;
    p.lse = a.lse; p.delta = a.delta; p.dq = a.dq; p.sq_b = a.sq.stride_b; p.sq_s = a.sq.stride_s; p.sq_h = a.sq.stride_h;
    p.dkv_acc = a.dkv_acc; p.status = device_status_word();
    p.q_col0_stride = (int)a.sq.stride_h; p.do_col0_stride = (int)a.sdo.stride_h;
    p.k_col0_stride = (int)a.sk.stride_h; p.v_col0_stride = (int)a.sv.stride_h;
    if (compute_delta) {
        if (a.so.stride_b % 8 || a.so.stride_s % 8 || a.so.stride_h % 8 || a.sdo.stride_b % 8 || a.sdo.stride_s % 8) return MFT_ERR_UNSUPPORTED;
        p.o = a.o; p.d_o = a.d_o; p.delta_out = a.delta;
        p.so_b = a.so.stride_b; p.so_s = a.so.stride_s; p.so_h = a.so.stride_h;
        p.sdo_b = a.sdo.stride_b; p.sdo_s = a.sdo.stride_s; p.sdo_h = a.sdo.stride_h;
    }
    dim3 grid((unsigned)(a.seq / BM), (unsigned)a.n_heads, (unsigned)a.batch);
    return HD_DISPATCH(hd, launch_dq<64>(mq, md, mk, mv, p, grid, stream), launch_dq<128>(mq, md, mk, mv, p, grid, stream), launch_dq<256>(mq, md, mk, mv, p, grid, stream));
}

int32_t attn_dkv_sm100(const AttnParams& a, int hd, cudaStream_t stream) {
    static const int enabled = [] { const char* e = std::getenv("MFT_ATTN_TC"); return e ? std::atoi(e) : 1; }();
    if (!enabled || !tc_shape_ok(hd) || a.seq % BM != 0 || !a.dkv_acc || !device_status_word()) return MFT_ERR_UNSUPPORTED;
    // the backward kernels win from 256 tokens on (0.064 against 0.073 ms at 256, 2.6 x at 4096); MFT_ATTN_TC=2 forces them
    if (hd != 256 && a.seq < 256 && enabled < 2) return MFT_ERR_UNSUPPORTED;
    if (!token_major(a.sq, a.seq) || !token_major(a.sk, a.seq) || !token_major(a.sv, a.seq) || !token_major(a.sdo, a.seq)) return MFT_ERR_UNSUPPORTED;
    if (a.sq.stride_h % 8 || a.sk.stride_h % 8 || a.sv.stride_h % 8 || a.sdo.stride_h % 8) return MFT_ERR_UNSUPPORTED;
    if ((int64_t)a.batch * a.seq >= (1ll << 31) || 2 * a.n_heads > 65535) return MFT_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(a.lse) % 16 || reinterpret_cast<uintptr_t>(a.delta) % 16 || reinterpret_cast<uintptr_t>(a.dkv_acc) % 16) return MFT_ERR_UNSUPPORTED;
    CUtensorMap mq, md, mk, mv;
    const int64_t rows = (int64_t)a.batch * a.seq;
    if (make_tmap_bf16(&mq, a.q, rows, (int64_t)(a.n_heads - 1) * a.sq.stride_h + hd, a.sq.stride_s, KV_BQ) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&md, a.d_o, rows, (int64_t)(a.n_heads - 1) * a.sdo.stride_h + hd, a.sdo.stride_s, KV_BQ) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mk, a.k, rows, (int64_t)(a.n_kv - 1) * a.sk.stride_h + hd, a.sk.stride_s, BM) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    if (make_tmap_bf16(&mv, a.v, rows, (int64_t)(a.n_kv - 1) * a.sv.stride_h + hd, a.sv.stride_s, BM) != MFT_OK) return MFT_ERR_UNSUPPORTED;
    BwdParams p{};
    p.seq = a.seq; p.n_heads = a.n_heads; p.n_kv = a.n_kv; p.rep = a.rep; p.window = a.window; p.scale = a.scale;
    p.lse = a.lse; p.delta = a.delta; p.dq = a.dq; p.sq_b = a.sq.stride_b; p.sq_s = a.sq.stride_s; p.sq_h = a.sq.stride_h;
    p.dkv_acc = a.dkv_acc; p.status = device_status_word();
    p.q_col0_stride = (int)a.sq.stride_h; p.do_col0_stride = (int)a.sdo.stride_h;
    p.k_col0_stride = (int)a.sk.stride_h; p.v_col0_stride = (int)a.sv.stride_h;
    return HD_DISPATCH(hd, launch_dkv<64>(mq, md, mk, mv, p, a.seq, a.n_heads, a.batch, stream), launch_dkv<128>(mq, md, mk, mv, p, a.seq, a.n_heads, a.batch, stream),
                       launch_dkv<256>(mq, md, mk, mv, p, a.seq, a.n_heads, a.batch, stream));
}

}  // namespace mft
