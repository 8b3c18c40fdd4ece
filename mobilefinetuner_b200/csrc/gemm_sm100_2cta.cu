// CTA-pair variant of the bf16 "NT" tcgen05 GEMM: two CTAs of a cluster (two SMs) cooperate on one
// 256 x 256 or 256 x 384 output tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and HALF
// of the B tile, so the shared-memory operand traffic per SM is 2/3 of the single-CTA kernel's (which is bound by
// it), while each SM's tensor memory holds the accumulator rows of its own half of the tile.  The main loop is bound by
// how fast operands arrive from L2, so the tile shape is chosen for operand bytes per output column (PairCfg).
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = tensor-memory allocation and - in the
// leader CTA (cluster rank 0) only - the one MMA-issuing thread, warps 2..9 = epilogue for this CTA's
// 128 rows, two warps per lane quadrant of tensor memory.  Barriers: `full` and `tmem_empty` live in the leader (both
// CTAs arrive there, the peer through the cluster shared-memory window); `empty` and `tmem_full` exist in both CTAs
// and are signalled for both by one tcgen05.commit.  TMA loads are plain per-CTA loads (each CTA fetches its
// own tiles; nothing is broadcast).  All waits are bounded, as in the single-CTA kernel.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

using namespace ptx;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int EPI_WARPS = 8;                  // two per lane quadrant of tensor memory: see BoxPair
constexpr int THREADS = 64 + 32 * EPI_WARPS;  // TMA warp, MMA warp, epilogue warps
constexpr int BAR_BYTES = 1024;               // barriers, tensor-memory slot, abort flag, per-quadrant row sums
constexpr int A_BYTES = BM * BK * 2;
constexpr int STORE_BYTES = 4 * 2 * EPI_BOX_BYTES;
// BN2 = columns of the pair's tile.  256 is the general width: 192 measured 17 % slower per column and 128
// 40 % slower (their operand loads per MMA cycle outrun what the L2 delivers), which costs more than the tile
// quantisation they would save.  Each CTA stages A (16 KB) and BN2/2 rows of B per k-block.
// BN2 = 384 (WIDE) goes the other way for outputs whose width is a multiple of 384 under a long K: one A tile then
// serves 384 columns (40 KB of operands per 256 x 384 x 64 block instead of 48 KB in 256-wide tiles, and no half-empty
// fifth column tile at N = 1152).  Its accumulator takes 384 of the 512 tensor-memory columns, so there is one
// accumulator buffer and the epilogue of a tile is not overlapped with the next tile's MMAs: it is used only where
// the K loop is long against the epilogue.  One k-step is two MMAs of 192 columns, each reading 96 B rows per CTA.
// The gated-MLP backward epilogue keeps GLU_SETS sets of (gate, up) boxes per warp (loaded by TMA, rewritten in place,
// stored by TMA): twice the box memory of the other epilogues, paid for with one pipeline stage.
// STAGED (wide tiles with a bf16 output): the epilogue first moves the whole accumulator of the CTA, rounded to bf16,
// into a 96 KB staging area of 24 swizzled boxes, hands the tensor memory back to the MMA issuer, and only then stores
// the boxes (and, for the gated MLP, forms f(gate) * up from the staged values), which overlaps with the next tile's
// K loop.  That keeps the exposed part of the epilogue short enough for K = 1152.  The staging area costs one pipeline
// stage (3 x 40 KB in flight measured 2 % slower than 4 on the long-K shapes).
template <int EPI, int BN2, bool STAGED>
struct PairCfg {
    static constexpr int BH_BYTES = (BN2 / 2) * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + BH_BYTES;                  // 32 / 40 KB, multiples of 1024
    static constexpr int STAGING_BYTES = BM * BN2 * 2;
    static constexpr int BOX_BYTES = EPI == EPI_GLU_BWD ? GLU_SETS * STORE_BYTES : (STAGED ? STAGING_BYTES : STORE_BYTES);
    static constexpr bool WIDE = BN2 > 256;
    static constexpr int ACC_BUFS = WIDE ? 1 : 2;
    static constexpr int MMA_N = WIDE ? BN2 / 2 : BN2;                      // columns of one MMA instruction (plain wide tile)
    static constexpr int STAGES = EPI == EPI_GLU_BWD ? 8 - GLU_SETS - 1 : (STAGED ? 3 : (WIDE ? 4 : 6));
    static_assert(!WIDE || BN2 == 384, "wide tiles are 384 columns");
    static_assert(!WIDE || EPI == EPI_STORE || (EPI == EPI_GLU_FWD && STAGED), "wide tiles: plain store, or the staged gated-MLP forward");
    static_assert(!STAGED || WIDE, "the staged epilogue belongs to the wide tile");
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BOX_BYTES + 1024 + BAR_BYTES;
};
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;   // clears the bit that distinguishes the two CTAs of a pair: -> address in the leader

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
// per-CTA tile load whose completion bytes are credited to a barrier in the leader CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_addr, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_addr), "r"(c0), "r"(c1)
        : "memory");
}
// named barrier 1 over the 8 epilogue warps; the second form also tells every thread whether `ok` held in all of them
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory"); }
__device__ __forceinline__ bool epi_barrier_and(bool ok) {
    uint32_t all;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(all)
        : "r"((uint32_t)ok), "n"(32 * EPI_WARPS)
        : "memory");
    return all != 0;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrive on the barrier at the same shared-memory offset in BOTH CTAs of the pair, once all prior MMAs are done
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int EPI, int BN2, bool STAGED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_nt_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                    const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    dep_trigger();
    using Cfg = PairCfg<EPI, BN2, STAGED>;
    constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int BOX_BYTES = Cfg::BOX_BYTES;
    constexpr bool WIDE = Cfg::WIDE;
    constexpr int ACC_BUFS = Cfg::ACC_BUFS, MMA_N = Cfg::MMA_N;
    constexpr bool GLU_FWD = EPI == EPI_GLU_FWD, GLU_BWD = EPI == EPI_GLU_BWD;
    // wide tile, per CTA 192 rows of B in two boxes of 96.  Plain: two MMAs of 192 columns, the pair's first takes B rows
    // 0..95 of each CTA (columns 0..191 of the tile), the second rows 96..191.  Gated MLP: the leader holds 192 gate rows,
    // the peer the 192 matching up rows; an MMA of 256 columns over rows 0..127 of each CTA (accumulator columns 0..127
    // gate, 128..255 up) and one of 128 columns over rows 128..191 (256..319 gate, 320..383 up) keep every 64-column
    // chunk of the accumulator on one side.
    constexpr int N_LO = !WIDE ? BN2 : (GLU_FWD ? 256 : MMA_N), N_HI = BN2 - N_LO;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* store_smem = tiles + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(store_smem + BOX_BYTES);
    uint64_t* full_bar = bars;                    // [STAGES]  used in the leader
    uint64_t* empty_bar = bars + STAGES;          // [STAGES]  both CTAs
    uint64_t* tmem_full_bar = bars + 2 * STAGES;  // [2]       both CTAs
    uint64_t* tmem_empty_bar = tmem_full_bar + 2; // [2]       used in the leader
    uint64_t* glu_bar = tmem_empty_bar + 2;       // [4 warps][GLU_SETS]  gated-MLP backward: gate / up boxes have landed
    uint64_t* pair_bar = glu_bar + 4 * GLU_SETS;  // [4 quadrants][free, filled, sums]: the two epilogue warps of a quadrant
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair_bar + 4 * 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* pair_sums = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + BAR_BYTES / 2);    // [4][32]
    static_assert((2 * 8 + 4 + 4 * GLU_SETS + 12) * 8 + 8 <= BAR_BYTES / 2, "barrier block");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int num_clusters = gridDim.x / 2, cluster_id = blockIdx.x / 2;
    const int num_tiles = p.tiles_mn * p.splits;                    // 256 x BN2 tiles, times the K ranges
    const int num_kb_main = (p.k + BK - 1) / BK;
    const int num_kb = num_kb_main + (p.k2 > 0 ? 1 : 0);            // splits > 1 only without the second segment

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full_bar[b], 1); mbar_init(&tmem_empty_bar[b], 2 * EPI_WARPS); }
        for (int b = 0; b < 4 * GLU_SETS; ++b) mbar_init(&glu_bar[b], 1);
        for (int b = 0; b < 4 * 3; ++b) mbar_init(&pair_bar[b], 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_a); tma_prefetch_desc(&map_b); tma_prefetch_desc(&map_d);
        if (GLU_FWD || GLU_BWD) tma_prefetch_desc(&map_x);
    }
    __syncthreads();
    if (warp == 1) { tmem_alloc2(tmem_slot, 512); tmem_relinquish2(); }
    tc_fence_before();
    cluster_sync();             // barrier inits of both CTAs are visible before anyone arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    dep_wait();     // set-up above overlapped the previous kernel's tail; its results are needed from here on

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
                const int t2 = tile % p.tiles_mn, split = tile / p.tiles_mn;
                const int m0 = tile_m(t2, p) * 2 * BM + (int)rank * BM;
                // the MMA of a ragged last column tile is narrowed to the columns that exist (rounded up to 16); a
                // pair MMA of width n_eff reads n_eff/2 rows of B from each CTA, so the halves are cut there
                const int n_base = tile_n(t2, p) * BN2;
                const int n_eff = min(BN2, (p.n - n_base + 15) & ~15);
                // gated-MLP forward: the leader loads 128 gate rows of the weight, the peer the 128 matching up rows
                // wide tile: the pair's first MMA takes columns 0..191 (96 B rows from each CTA), the second 192..383
                const int n0 = GLU_FWD ? tile_n(t2, p) * (BN2 / 2) + (int)rank * p.glu_inter
                             : WIDE ? n_base + (int)rank * (MMA_N / 2) : n_base + (int)rank * (n_eff / 2);
                const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sa = tiles + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    const uint32_t full_in_leader = smem_u32(&full_bar[stage]) & PEER_MASK;
                    mbar_arrive_expect_tx_cluster(full_in_leader, STAGE_BYTES);
                    const CUtensorMap* ta = kb < num_kb_main ? &map_a : &map_a2;
                    const CUtensorMap* tb = kb < num_kb_main ? &map_b : &map_b2;
                    const int k0 = kb < num_kb_main ? kb * BK : 0;
                    tma_load_2d_pair(sa, ta, full_in_leader, k0, m0);
                    tma_load_2d_pair(sb, tb, full_in_leader, k0, n0);
                    if (WIDE) tma_load_2d_pair(sb + (BN2 / 4) * BK * 2, tb, full_in_leader, k0, n0 + (GLU_FWD ? BN2 / 4 : MMA_N));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
                const int acc = ACC_BUFS == 2 ? it & 1 : 0;
                const uint32_t acc_phase = ACC_BUFS == 2 ? (it >> 1) & 1 : it & 1;
                if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN2;
                const int split = tile / p.tiles_mn;
                const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
                const int n_base = tile_n(tile % p.tiles_mn, p) * BN2;
                const uint32_t idesc = idesc_bf16_f32(2 * BM, WIDE ? (uint32_t)N_LO : GLU_FWD ? (uint32_t)BN2 : (uint32_t)min(BN2, (p.n - n_base + 15) & ~15));
                const uint32_t idesc_hi = idesc_bf16_f32(2 * BM, WIDE ? (uint32_t)N_HI : 16u);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + A_BYTES);
                    const int kvalid = (kb < num_kb_main) ? min(BK, p.k - kb * BK) : p.k2;
                    const int nmma = (kvalid + 15) / 16;
                    if (STAGED && kb == kb0) {
                        // first k-block of a tile: the second MMA's columns come back from the epilogue after the first's.
                        // (This wait sits outside the loop that issues the MMAs: with a conditional wait inside that loop
                        // every k-block of the call measured 40 % slower.)
                        for (int j = 0; j < nmma; ++j)
                            umma2_bf16(tmem_d, adesc + (uint64_t)(2 * j), bdesc + (uint64_t)(2 * j), idesc, j != 0 ? 1u : 0u);
                        if (!mbar_wait(&tmem_empty_bar[1], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t bdesc_hi = smem_desc_sw128(sa + A_BYTES + (N_LO / 2) * BK * 2);
                        for (int j = 0; j < nmma; ++j)
                            umma2_bf16(tmem_d + N_LO, adesc + (uint64_t)(2 * j), bdesc_hi + (uint64_t)(2 * j), idesc_hi, j != 0 ? 1u : 0u);
                    } else {
                        for (int j = 0; j < nmma; ++j) {
                            umma2_bf16(tmem_d, adesc + (uint64_t)(2 * j), bdesc + (uint64_t)(2 * j), idesc, (kb > kb0 || j != 0) ? 1u : 0u);
                            if (WIDE) {
                                const uint64_t bdesc_hi = smem_desc_sw128(sa + A_BYTES + (N_LO / 2) * BK * 2);
                                umma2_bf16(tmem_d + N_LO, adesc + (uint64_t)(2 * j), bdesc_hi + (uint64_t)(2 * j), idesc_hi, (kb > kb0 || j != 0) ? 1u : 0u);
                            }
                        }
                    }
                    umma2_commit_both(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma2_commit_both(&tmem_full_bar[acc]);
            }
        }
    } else if constexpr (STAGED) {
        // ------------------------------------------------ staged epilogue of the wide tile (see PairCfg)
        const int q = warp & 3, ew = warp - 2, side = ew >> 2;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        int it = 0;
        for (int tile = cluster_id; tile < num_tiles; tile += num_clusters, ++it) {
            const int t2 = tile % p.tiles_mn;
            const int m0 = tile_m(t2, p) * 2 * BM + (int)rank * BM;
            const int n0 = GLU_FWD ? tile_n(t2, p) * (BN2 / 2) : tile_n(t2, p) * BN2;
            const bool landed = mbar_wait(&tmem_full_bar[0], (uint32_t)(it & 1), abort_flag);
            if (lane == 0) tma_store_wait_read<0>();       // this warp's stores of the previous tile have read their boxes
            // every epilogue warp is here: the staging area is free, and all of them go on or all of them stop
            if (!epi_barrier_and(landed)) break;
            tc_fence_after();
            // the columns of the tile's first MMA are handed back first (barrier 0), the second MMA's after them (1)
            constexpr int LO_CHUNKS = N_LO / 64;
            staged_drain<EPI, 0, LO_CHUNKS>(p, store_smem, taddr, q, side, lane, n0);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tmem_empty_bar[0]) & PEER_MASK);   // count: 8 warps x 2 CTAs
            staged_drain<EPI, LO_CHUNKS, 6>(p, store_smem, taddr, q, side, lane, n0);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tmem_empty_bar[1]) & PEER_MASK);
            fence_proxy_async();
            epi_barrier();                                 // the whole staging area is written
            if constexpr (GLU_FWD) staged_store_glu(p, &map_d, &map_x, store_smem, ew, lane, m0, n0);
            else staged_store_plain(&map_d, store_smem, ew, lane, m0, n0, p.n);
        }
        if (lane == 0) tma_store_wait<0>();
    } else {
        // ------------------------------------------------ epilogue: this CTA's 128 rows of the pair tile
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        int it = 0, box_ctr = 0;
        bool ok = true;
        BoxPair bp;
        bp.free_bar = pair_bar + q * 3; bp.filled_bar = bp.free_bar + 1; bp.sum_bar = bp.free_bar + 2;
        bp.sums = pair_sums + q * 32;
        bp.abort_flag = abort_flag;
        bp.side = (warp - 2) >> 2;                                // warps 2..5 own the boxes of quadrants 2, 3, 0, 1; warps 6..9 help
        GluBwdState glu_state;
        if (GLU_BWD) {                                            // gate / up boxes of this quadrant's first chunk(s)
            glu_state.ahead_tile = cluster_id;
            if (lane == 0 && bp.side == 0)
                for (int i = 0; i < GLU_SETS - 1; ++i) glu_bwd_prefetch(p, &map_x, store_smem, glu_bar, q, (int)rank, num_clusters, num_tiles, glu_state);
        }
        for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
            const int acc = ACC_BUFS == 2 ? it & 1 : 0;
            const uint32_t acc_phase = ACC_BUFS == 2 ? (it >> 1) & 1 : it & 1;
            const int t2 = tile % p.tiles_mn;
            const int m0 = tile_m(t2, p) * 2 * BM + (int)rank * BM;
            const int n0 = GLU_FWD ? tile_n(t2, p) * (BN2 / 2) : tile_n(t2, p) * BN2;
            if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + row_in_tile;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN2);
            if constexpr (GLU_FWD) {
                ok = epilogue_glu_fwd(p, &map_d, &map_x, store_smem, taddr, q, lane, m0 + q * 32, n0, box_ctr, bp);
            } else if constexpr (GLU_BWD) {
                ok = epilogue_glu_bwd(p, &map_d, &map_x, store_smem, glu_bar, abort_flag, taddr, q, lane, (int)rank, m0 + q * 32, n0, num_clusters,
                                      num_tiles, glu_state, bp);
            } else
            if (EPI == EPI_STORE && p.d_is_f32)
                ok = epilogue_f32_tma<BN2>(p, &map_d, store_smem, taddr, q, lane, m0 + q * 32, n0, p.bias != nullptr && tile < p.tiles_mn, box_ctr, bp);
            else
                ok = epilogue_bf16_tma<EPI, BN2>(p, &map_d, store_smem, taddr, q, lane, row, m0 + q * 32, n0, box_ctr, bp);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tmem_empty_bar[acc]) & PEER_MASK);   // the accumulator buffer is free (count: 8 warps x 2 CTAs)
        }
        if (lane == 0) tma_store_wait<0>();
    }

    // ------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, MFT_ERR_TIMEOUT);
    cluster_sync();             // the peer may still be read by the leader's MMAs / written by its commits until here
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

template <int EPI, int BN2, bool STAGED = false>
int32_t launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma2, const CUtensorMap& mb2, const CUtensorMap& md,
               const CUtensorMap& mx, GemmParams p, cudaStream_t stream) {
    using Cfg = PairCfg<EPI, BN2, STAGED>;
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(gemm_nt_2cta_kernel<EPI, BN2, STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES), "gemm 2cta smem attr")) return s;
        configured = true;
    }
    const int tiles = p.tiles_mn * p.splits;
    int clusters = num_sms() / 2;
    if (tiles < clusters) clusters = tiles;
    launch_dep(gemm_nt_2cta_kernel<EPI, BN2, STAGED>, dim3(2 * clusters), dim3(THREADS), (size_t)(Cfg::SMEM_BYTES), stream, ma, mb, ma2, mb2, md, mx, p);
    MFT_LAUNCH_CHECK("gemm_nt_2cta");
    return MFT_OK;
}

// Cost of a call in units of one k-block of a 256 x 256 tile: waves of tiles over the clusters times the k-blocks of a
// tile (plus a per-tile charge), each extra K range charged 0.2 % for its pass over D.  A k-block of a 384-wide tile
// measured 1.25 of a 256-wide one for 1.5 times the columns (0.643 against 0.515 us at 16384 x 1152 x 6912 and
// x 13824).  Its per-tile charge: the streaming epilogue of the f32 output (about 7000 clocks) is not overlapped; the
// staged one leaves a gap of about 3000 clocks in which no operand requests are in flight.  A ragged last column tile
// counts as a full one: narrowing its MMAs was measured to save nothing, the main loop is bound by operand delivery.
struct TileShape { int64_t m_tiles, n_tiles; bool wide, staged; };
double tile_cost(const TileShape& t, int64_t kb, int sp) {
    const int64_t clusters = num_sms() / 2;
    const int64_t per = (kb + sp - 1) / sp, waves = (t.m_tiles * t.n_tiles * sp + clusters - 1) / clusters;
    const double unit = t.wide ? 1.25 : 1.0, per_tile = t.wide ? (t.staged ? 6.5 : 11.0) : 4.0;
    return (double)waves * ((double)per * unit + per_tile) * (1.0 + 0.002 * (sp - 1));
}
// Number of K ranges for an f32 output whose caller leaves the choice open, and the cost of that choice.
int choose_splits(const TileShape& t, int64_t kb, double* cost_out) {
    int best_sp = 1;
    double best = 1e300;
    for (int sp = 1; sp <= 8; ++sp) {
        if (sp > 1 && kb / sp < (t.wide ? 64 : 32)) break;
        const double cost = tile_cost(t, kb, sp);
        if (cost < best * 0.995) { best = cost; best_sp = sp; }
    }
    if (cost_out) *cost_out = best;
    return best_sp;
}

// Tile width (256 or 384 columns) and number of K ranges of a call.  n_tiles_wide = 0: the call has no whole 384-column
// tiles.  `staged`: bf16 output (the wide tile's epilogue is the staged one; otherwise its K loop must be at least
// 64 blocks long).  `asked` = the caller's K ranges, 0 = choose.  MFT_GEMM_WIDE=0 keeps every call on 256-wide tiles.
int plan_tiles(int64_t m, int64_t n_tiles, int64_t n_tiles_wide, int64_t kb, bool staged, bool can_split, int asked, int* splits_out, bool ragged = false) {
    static const bool wide_allowed = [] { const char* e = std::getenv("MFT_GEMM_WIDE"); return !(e && e[0] == '0'); }();
    const TileShape t256{(m + 255) / 256, n_tiles, false, false}, t384{(m + 255) / 256, n_tiles_wide, true, staged};
    const bool wide_fits = wide_allowed && n_tiles_wide > 0 && m % 256 == 0;
    bool wide = false;
    int splits = 1;
    const double margin = ragged ? 0.97 : 1.0;        // a ragged last tile computes columns that do not exist: ask for a clear gain
    if (!can_split || asked > 0) {
        splits = can_split ? asked : 1;
        wide = wide_fits && (staged || kb / splits >= 64) && tile_cost(t384, kb, splits) < margin * tile_cost(t256, kb, splits);
    } else {
        double cost256 = 0, cost384 = 0;
        const int sp256 = choose_splits(t256, kb, &cost256);
        const int sp384 = wide_fits && (staged || kb >= 64) ? choose_splits(t384, kb, &cost384) : 0;
        wide = sp384 > 0 && cost384 < margin * cost256;
        splits = wide ? sp384 : sp256;
    }
    *splits_out = splits;
    return wide ? 384 : 256;
}

}  // namespace

// what gemm_nt_run_2cta would choose for a plain-store call of this shape (0 when the pair kernel does not take it)
int gemm_nt_pair_tile_cols(int64_t m, int64_t n, int64_t k, int64_t k2, bool d_is_f32) {
    if (m < 256 || n < 192) return 0;
    const int64_t kb = (k + BK - 1) / BK + (k2 > 0 ? 1 : 0);
    int splits = 1;
    return plan_tiles(m, (n + 255) / 256, n >= 384 ? (n + 383) / 384 : 0, kb, !d_is_f32, d_is_f32 && k2 == 0, 0, &splits, n % 384 != 0);
}

int32_t gemm_nt_run_2cta(const GemmCall& c, cudaStream_t stream) {
    const bool ce = c.epi == EPI_CE_GRAD || c.epi == EPI_CE_P;
    const bool glu = c.epi == EPI_GLU_FWD || c.epi == EPI_GLU_BWD;
    const bool bf16_ok = !c.d_is_f32 && !c.accumulate && (c.ldd % 8 == 0);
    const bool f32_ok = c.d_is_f32 && c.epi == EPI_STORE && (c.ldd % 4 == 0);
    const bool ok = (c.epi == EPI_STORE || ce || glu) && (bf16_ok || f32_ok) && c.d && (reinterpret_cast<uintptr_t>(c.d) % 16 == 0) &&
                    c.m >= 256 && c.n >= 192 && c.splits >= 0 && c.splits <= 64;
    if (!ok) return MFT_ERR_UNSUPPORTED;
    if (glu) {
        // forward: n = 2 * inter columns of D, tiles of 128 gate + 128 up columns; backward: n = inter
        const int64_t inter = c.glu_inter;
        const bool shape_ok = c.epi == EPI_GLU_FWD ? (c.n == 2 * inter && inter % 128 == 0) : (c.n == inter && inter % 64 == 0);
        if (!shape_ok || !c.aux || c.ld_aux % 8 != 0 || reinterpret_cast<uintptr_t>(c.aux) % 16 != 0 || c.d_is_f32 || inter >= (1 << 30))
            return MFT_ERR_UNSUPPORTED;
    }
    const bool can_split = f32_ok && c.k2 == 0;
    if (c.splits > 1 && !can_split) return MFT_ERR_UNSUPPORTED;
    const int64_t kb = (c.k + BK - 1) / BK + (c.k2 > 0 ? 1 : 0);
    // the wide tile: plain store or gated-MLP forward over whole 384-column tiles, when the cost model prefers it (a call
    // of a few tiles is one wave either way, and the wave of wide tiles is the longer one)
    int splits = 1;
    int bn = 256;
    // a ragged last 384-column tile is computed whole (the rows of B past N arrive as zeros) and stored clipped
    if (c.epi == EPI_STORE) bn = plan_tiles(c.m, (c.n + 255) / 256, c.n >= 384 ? (c.n + 383) / 384 : 0, kb, bf16_ok, can_split, (int)c.splits, &splits, c.n % 384 != 0);
    else if (c.epi == EPI_GLU_FWD) bn = plan_tiles(c.m, c.glu_inter / 128, c.glu_inter % 192 == 0 ? c.glu_inter / 192 : 0, kb, true, false, 0, &splits);
    const bool wide = bn > 256;
    CUtensorMap ma, mb, ma2, mb2, md, mx;
    if (int32_t s = make_tmap_bf16(&ma, c.a, c.m, c.k, c.lda, BM)) return s;
    const int b_box = wide ? 96 : 128;                 // B rows per box: see the producer
    if (int32_t s = make_tmap_bf16(&mb, c.b, c.n, c.k, c.ldb, b_box)) return s;
    if (c.k2 > 0) {
        if (int32_t s = make_tmap_bf16(&ma2, c.a2, c.m, c.k2, c.lda2, BM)) return s;
        if (int32_t s = make_tmap_bf16(&mb2, c.b2, c.n, c.k2, c.ldb2, b_box)) return s;
    } else {
        ma2 = ma; mb2 = mb;
    }
    if (c.d_is_f32) {
        if (int32_t s = make_tmap_f32_out(&md, c.d, c.m, c.n, c.ldd)) return s;
    } else {
        // the gated-MLP backward writes d_gate|d_up: D is twice as wide as the GEMM
        if (int32_t s = make_tmap_bf16(&md, c.d, c.m, c.epi == EPI_GLU_BWD ? 2 * c.n : c.n, c.ldd, 32)) return s;
    }
    mx = md;
    if (c.epi == EPI_GLU_FWD) { if (int32_t s = make_tmap_bf16(&mx, c.aux, c.m, c.glu_inter, c.ld_aux, 32)) return s; }
    if (c.epi == EPI_GLU_BWD) { if (int32_t s = make_tmap_bf16(&mx, c.aux, c.m, 2 * c.glu_inter, c.ld_aux, 32)) return s; }
    GemmParams p{};
    p.m = (int)c.m; p.n = (int)c.n; p.k = (int)c.k; p.k2 = (int)c.k2;
    p.alpha = c.alpha; p.bias = c.bias; p.d = c.d; p.ldd = c.ldd; p.tma_store = 1;
    p.d_is_f32 = c.d_is_f32; p.accumulate = c.accumulate; p.f32_reduce = (c.d_is_f32 && c.accumulate) ? 1 : 0;
    p.status = device_status_word();
    p.ce_tgt = c.ce_tgt; p.ce_lse = c.ce_lse; p.ce_nvalid = c.ce_nvalid; p.ce_nvalid_override = c.ce_nvalid_override;
    p.ce_dloss = c.ce_dloss; p.ce_col_offset = c.ce_col_offset;
    p.ce_partials = c.ce_partials; p.ce_partial_ld = c.ce_partial_ld; p.ce_tgt_logit = c.ce_tgt_logit; p.ce_flag = c.ce_flag;
    p.glu_geglu = c.glu_geglu; p.glu_inter = (int)c.glu_inter;
    p.num_m_tiles = (p.m + 2 * BM - 1) / (2 * BM);
    p.num_n_tiles = c.epi == EPI_GLU_FWD ? (int)(c.glu_inter / (bn / 2)) : (p.n + bn - 1) / bn;
    p.tiles_mn = p.num_m_tiles * p.num_n_tiles;
    p.kb_per_split = (int)((kb + splits - 1) / splits);
    p.splits = (int)((kb + p.kb_per_split - 1) / p.kb_per_split);
    if (p.splits > 1 && !p.f32_reduce) {
        if (int32_t s = check_cuda(cudaMemset2DAsync(p.d, (size_t)p.ldd * 4, 0, (size_t)p.n * 4, (size_t)p.m, stream), "gemm split-K memset")) return s;
        p.f32_reduce = 1;
    }
    if (c.epi == EPI_CE_GRAD) return launch<EPI_CE_GRAD, 256>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (c.epi == EPI_CE_P) return launch<EPI_CE_P, 256>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (c.epi == EPI_GLU_FWD && wide) return launch<EPI_GLU_FWD, 384, true>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (c.epi == EPI_GLU_FWD) return launch<EPI_GLU_FWD, 256>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (c.epi == EPI_GLU_BWD) return launch<EPI_GLU_BWD, 256>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (wide && !c.d_is_f32) return launch<EPI_STORE, 384, true>(ma, mb, ma2, mb2, md, mx, p, stream);
    if (wide) return launch<EPI_STORE, 384>(ma, mb, ma2, mb2, md, mx, p, stream);
    return launch<EPI_STORE, 256>(ma, mb, ma2, mb2, md, mx, p, stream);
}

}  // namespace mft
