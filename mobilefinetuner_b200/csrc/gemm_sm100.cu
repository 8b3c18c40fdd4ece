// bf16 "NT" GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a:
//     D[m,n] = alpha * ( A[m,:K].B[n,:K] + A2[m,:K2].B2[n,:K2] ) + bias[n] (+ D[m,n])
// The second (A2,B2) segment carries the rank-r LoRA update in the same
// accumulator (A2 = scale*(X*A), B2 = B^T), see include/mft_cuda.h.
//
// Structure: persistent kernel, one CTA per SM, 128 x BLOCK_N output tiles,
// 64-wide k-blocks.  Warp 0 = TMA producer (cp.async.bulk.tensor into a
// multi-stage shared-memory ring, 128-byte swizzle), warp 1 = MMA issuer (one
// thread issues tcgen05.mma, accumulators live in tensor memory, two
// accumulator buffers so the epilogue of tile i overlaps the main loop of tile
// i+1), warps 2..5 = epilogue (tcgen05.ld -> registers -> alpha/bias/convert ->
// global).  All mbarrier waits are bounded; a wait that runs out sets the
// library status word to MFT_ERR_TIMEOUT and the CTA leaves after freeing its
// tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace mft {

using namespace ptx;

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;



template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
    static constexpr int B_BYTES = BN * GEMM_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 4 : (BN == 128 ? 6 : 8));
    static constexpr int TMEM_COLS = (BN > 128) ? 512 : 2 * BN;     // two accumulators; a power of two >= 32
    static constexpr int STORE_BOX_BYTES = 32 * 64 * 2;               // 32 rows x 64 bf16 columns
    static constexpr int STORE_BYTES = 4 * 2 * STORE_BOX_BYTES;       // 4 epilogue warps x 2 buffers
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_nt_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
               const __grid_constant__ CUtensorMap map_d, const GemmParams p) {
    dep_trigger();
    using Cfg = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms (8 rows x 128 B)
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* store_smem = tiles + Cfg::STAGES * Cfg::STAGE_BYTES;   // 1024-byte aligned: STAGE_BYTES is a multiple of 1024
    uint64_t* bars = reinterpret_cast<uint64_t*>(store_smem + Cfg::STORE_BYTES);
    uint64_t* full_bar = bars;                         // [STAGES]
    uint64_t* empty_bar = bars + Cfg::STAGES;          // [STAGES]
    uint64_t* tmem_full_bar = bars + 2 * Cfg::STAGES;  // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;      // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_mn * p.splits;
    const int num_kb_main = (p.k + GEMM_BK - 1) / GEMM_BK;
    const int num_kb = num_kb_main + (p.k2 > 0 ? 1 : 0);     // splits > 1 only without the second segment

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full_bar[b], 1); mbar_init(&tmem_empty_bar[b], 4); }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (p.k2 > 0) { tma_prefetch_desc(&map_a2); tma_prefetch_desc(&map_b2); }
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    dep_wait();     // set-up above overlapped the previous kernel's tail; its results are needed from here on

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int t2 = tile % p.tiles_mn, split = tile / p.tiles_mn;
                const int m0 = tile_m(t2, p) * GEMM_BM;
                const int n0 = tile_n(t2, p) * BN;
                const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
                    uint8_t* sb = sa + Cfg::A_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                    if (kb < num_kb_main) {
                        tma_load_2d(sa, &map_a, &full_bar[stage], kb * GEMM_BK, m0);
                        tma_load_2d(sb, &map_b, &full_bar[stage], kb * GEMM_BK, n0);
                    } else {
                        tma_load_2d(sa, &map_a2, &full_bar[stage], 0, m0);
                        tma_load_2d(sb, &map_b2, &full_bar[stage], 0, n0);
                    }
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // give loads still in flight a bounded chance to land before the CTA leaves
                for (int s = 0; s < Cfg::STAGES; ++s)
                    for (int i = 0; i < 4096 && !mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                const int split = tile / p.tiles_mn;
                const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
                // a ragged last column tile issues narrower MMAs (existing columns rounded up to 16)
                const int n_left = p.n - tile_n(tile % p.tiles_mn, p) * BN;
                const uint32_t idesc = idesc_bf16_f32(GEMM_BM, (uint32_t)min(BN, (n_left + 15) & ~15));
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sb);
                    const int kvalid = (kb < num_kb_main) ? min(GEMM_BK, p.k - kb * GEMM_BK) : p.k2;
                    const int nmma = (kvalid + 15) / 16;
                    for (int j = 0; j < nmma; ++j) {
                        // advance 16 bf16 = 32 bytes along K inside the swizzle atom: +2 in 16-byte units
                        umma_bf16(tmem_d, adesc + (uint64_t)(2 * j), bdesc + (uint64_t)(2 * j), idesc, (kb > kb0 || j != 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);   // frees the stage once these MMAs have read it
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(&tmem_full_bar[acc]);
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                    // tensor-memory lane quarter this warp may read
        const int row_in_tile = q * 32 + lane;
        int it = 0;
        int box_ctr = 0;
        bool ok = true;
        BoxPair solo;                              // one warp per lane quarter: it fills whole boxes
        const bool vec_ok = p.d_is_f32 ? ((p.ldd % 4) == 0 && (reinterpret_cast<uintptr_t>(p.d) % 16) == 0)
                                       : ((p.ldd % 8) == 0 && (reinterpret_cast<uintptr_t>(p.d) % 16) == 0);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int t2 = tile % p.tiles_mn;
            const int m0 = tile_m(t2, p) * GEMM_BM;
            const int n0 = tile_n(t2, p) * BN;
            if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + row_in_tile;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            if (EPI == EPI_STORE && p.tma_store && p.d_is_f32) {
                epilogue_f32_tma<BN>(p, &map_d, store_smem, taddr, q, lane, m0 + q * 32, n0, p.bias != nullptr && tile < p.tiles_mn, box_ctr, solo);
            } else if (EPI != EPI_CE_STATS && p.tma_store) {
                epilogue_bf16_tma<EPI, BN>(p, &map_d, store_smem, taddr, q, lane, row, m0 + q * 32, n0, box_ctr, solo);
            } else if constexpr (EPI == EPI_STORE) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (n0 + c >= p.n) break;          // uniform across the warp
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)c, r);
                    tmem_ld_wait();
                    if (row < p.m) {
                        const int col0 = n0 + c;
                        const bool full = vec_ok && (col0 + 32 <= p.n);
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
                        if (p.bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (col0 + j < p.n) v[j] += __ldg(p.bias + col0 + j);
                        }
                        if (p.d_is_f32) {
                            float* drow = static_cast<float*>(p.d) + (long long)row * p.ldd + col0;
                            if (full) {
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                    if (p.accumulate) {
                                        const float4 prev = *reinterpret_cast<const float4*>(drow + j);
                                        o.x += prev.x; o.y += prev.y; o.z += prev.z; o.w += prev.w;
                                    }
                                    *reinterpret_cast<float4*>(drow + j) = o;
                                }
                            } else {
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + j < p.n) drow[j] = v[j] + (p.accumulate ? drow[j] : 0.f);
                            }
                        } else {
                            __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + col0;
                            if (full) {
#pragma unroll
                                for (int j = 0; j < 32; j += 8) {
                                    float t[8];
#pragma unroll
                                    for (int e = 0; e < 8; ++e) t[e] = v[j + e];
                                    store8(drow + j, t);
                                }
                            } else {
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + j < p.n) drow[j] = f32_to_bf16(v[j]);
                            }
                        }
                    }
                }
            } else if constexpr (EPI == EPI_CE_STATS) {
                const int tgt = (row < p.m) ? p.ce_tgt[row] - p.ce_col_offset : -1;
                float mx = -INFINITY, sum = 0.f;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (n0 + c >= p.n) break;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)c, r);
                    tmem_ld_wait();
                    const int col0 = n0 + c;
                    float cm = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float v = __uint_as_float(r[j]) * p.alpha;
                        if (col0 + j >= p.n) v = -INFINITY;
                        r[j] = __float_as_uint(v);
                        cm = fmaxf(cm, v);
                    }
                    if (tgt >= col0 && tgt < col0 + 32 && row < p.m) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (col0 + j == tgt) p.ce_tgt_logit[row] = __uint_as_float(r[j]);
                    }
                    const float nm = fmaxf(mx, cm);
                    float cs = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) cs += __expf(__uint_as_float(r[j]) - nm);
                    sum = sum * __expf(mx - nm) + cs;     // mx = -inf on the first chunk -> factor 0
                    mx = nm;
                }
                if (row < p.m) p.ce_partials[(long long)row * p.ce_partial_ld + (p.ce_col_offset + n0) / BN] = make_float2(mx, sum);
            } else {
                float lse = 0.f, coef = 0.f;
                int tgt = -1;
                if (row < p.m) {
                    tgt = p.ce_tgt[row];
                    lse = p.ce_lse[row];
                    const long long nv = p.ce_nvalid_override > 0 ? p.ce_nvalid_override : (long long)*p.ce_nvalid;
                    coef = (tgt >= 0 && nv > 0) ? p.ce_dloss / (float)nv : 0.f;
                    tgt -= p.ce_col_offset;
                }
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (n0 + c >= p.n) break;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)c, r);
                    tmem_ld_wait();
                    if (row < p.m) {
                        const int col0 = n0 + c;
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float pr = __expf(__uint_as_float(r[j]) * p.alpha - lse);
                            v[j] = (pr - (col0 + j == tgt ? 1.f : 0.f)) * coef;
                        }
                        __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + col0;
                        if (vec_ok && col0 + 32 <= p.n) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float t[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) t[e] = v[j + e];
                                store8(drow + j, t);
                            }
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.n) drow[j] = f32_to_bf16(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        if (lane == 0) tma_store_wait<0>();   // every tensor store of this warp has completed
    }

    // ------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, MFT_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

static EncodeTiledFn get_encode() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    });
    return g_encode;
}

// Tensor map over a row-major bf16 matrix [rows, cols] (row stride ld elements),
// box = {64 columns, box_rows rows}, 128-byte swizzle, zero fill outside.
// A tensor map is a pure function of (type, base, extents, stride, box): encoding one costs a driver call of a
// microsecond or two, and a GEMM launch needs three to six.  Each host thread keeps the maps it has encoded in a small
// direct-mapped table; a map stays valid when its memory is freed and handed out again (it holds an address and a
// geometry, nothing else).
struct TmapKey {
    const void* base; int64_t rows, cols, ld; int32_t box_rows, kind;
    bool operator==(const TmapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && kind == o.kind; }
};
struct TmapSlot { TmapKey key; CUtensorMap map; bool used; };
constexpr int TMAP_SLOTS = 2048;
static TmapSlot* tmap_slot(const TmapKey& k) {
    thread_local std::vector<TmapSlot> table(TMAP_SLOTS, TmapSlot{{nullptr, 0, 0, 0, 0, 0}, {}, false});
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
    h = (h ^ (uint64_t)k.rows * 0x9E3779B97F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
    h = (h ^ (uint64_t)k.cols * 0x94D049BB133111EBull ^ (uint64_t)k.ld * 0xD6E8FEB86659FD93ull ^ (uint64_t)(k.box_rows * 7 + k.kind)) * 0x9E3779B97F4A7C15ull;
    return &table[(size_t)((h >> 40) % TMAP_SLOTS)];
}

int32_t make_tmap_bf16(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    const TmapKey key{base, rows, cols, ld, box_rows, 0};
    TmapSlot* slot = tmap_slot(key);
    if (slot->used && slot->key == key) { *map = slot->map; return MFT_OK; }
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(MFT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return fail(MFT_ERR_INVALID_ARG, "GEMM operand base must be 16-byte aligned");
    if (ld % 8 != 0) return fail(MFT_ERR_INVALID_ARG, "GEMM operand row stride must be a multiple of 8 elements");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MFT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    slot->key = key; slot->map = *map; slot->used = true;
    return MFT_OK;
}

// Tensor map over a row-major f32 matrix [rows, cols]: box = {32 columns, 32 rows}, 128-byte swizzle.
int32_t make_tmap_f32_out(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld) {
    const TmapKey key{base, rows, cols, ld, 32, 1};
    TmapSlot* slot = tmap_slot(key);
    if (slot->used && slot->key == key) { *map = slot->map; return MFT_OK; }
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(MFT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MFT_ERR_CUDA, "cuTensorMapEncodeTiled (f32 output) failed with code " + std::to_string((int)r));
    slot->key = key; slot->map = *map; slot->used = true;
    return MFT_OK;
}

static int g_num_sms = 0;
int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    return g_num_sms;
}

template <int BN, int EPI>
static int32_t launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma2, const CUtensorMap& mb2, const CUtensorMap& md,
                           GemmParams p, cudaStream_t stream) {
    using Cfg = GemmCfg<BN>;
    static PerDeviceFlag configured_on;           // function attributes are per device
    bool& configured = configured_on.here();
    if (!configured) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(gemm_nt_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES), "gemm smem attr")) return s;
        configured = true;
    }
    p.num_m_tiles = (p.m + GEMM_BM - 1) / GEMM_BM;
    p.num_n_tiles = (p.n + BN - 1) / BN;
    p.tiles_mn = p.num_m_tiles * p.num_n_tiles;
    const int num_kb = (p.k + GEMM_BK - 1) / GEMM_BK + (p.k2 > 0 ? 1 : 0);
    if (p.splits == 0) {
        // choose the K split that fills the last wave best (each range keeps >= 32 k-blocks)
        double best = 0.0;
        p.splits = 1;
        for (int sp = 1; sp <= 8 && num_kb / sp >= 32; ++sp) {
            const long long t = (long long)p.tiles_mn * sp, waves = (t + num_sms() - 1) / num_sms();
            const double eff = (double)t / (double)(waves * num_sms());
            if (eff > best + 0.02) { best = eff; p.splits = sp; }
        }
    }
    p.kb_per_split = (num_kb + p.splits - 1) / p.splits;
    p.splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;       // no empty range
    if (p.splits > 1 && !p.f32_reduce) {
        // the partial tiles are added into D: start from zero
        if (int32_t s = check_cuda(cudaMemset2DAsync(p.d, (size_t)p.ldd * 4, 0, (size_t)p.n * 4, (size_t)p.m, stream), "gemm split-K memset")) return s;
        p.f32_reduce = 1;
    }
    const int tiles = p.tiles_mn * p.splits;
    const int grid = tiles < num_sms() ? tiles : num_sms();
    launch_dep(gemm_nt_kernel<BN, EPI>, dim3(grid), dim3(GEMM_THREADS), (size_t)(Cfg::SMEM_BYTES), stream, ma, mb, ma2, mb2, md, p);
    MFT_LAUNCH_CHECK("gemm_nt");
    return MFT_OK;
}

static int pick_bn(int64_t n) {
    // padded columns weighted by a rough per-tile efficiency: wide tiles amortise the A loads
    const int cand[4] = {256, 192, 128, 64};
    const double eff[4] = {1.0, 1.05, 1.5, 2.5};   // narrow tiles are bound by shared-memory operand traffic
    int best = 256; double best_cost = 1e30;
    for (int i = 0; i < 4; ++i) {
        const double cost = (double)((n + cand[i] - 1) / cand[i] * cand[i]) * eff[i];
        if (cost < best_cost) { best_cost = cost; best = cand[i]; }
    }
    return best;
}

// ---- optional per-launch timing (bench / profiling only): CUDA events around every GEMM launch
struct ProfEntry { cudaEvent_t e0, e1; double flops; int epi; int64_t m, n, k, k2; int d_is_f32; };
static std::vector<ProfEntry> g_prof;
static bool g_prof_on = false;

static int32_t gemm_nt_run_inner(const GemmCall& c, cudaStream_t stream);

bool gemm_profiling_enabled() { return g_prof_on; }

int32_t gemm_nt_run(const GemmCall& c, cudaStream_t stream) {
    if (!g_prof_on) return gemm_nt_run_inner(c, stream);
    ProfEntry e;
    cudaEventCreate(&e.e0); cudaEventCreate(&e.e1);
    e.flops = 2.0 * (double)c.m * (double)c.n * ((double)c.k + (double)c.k2);
    e.epi = c.epi; e.m = c.m; e.n = c.n; e.k = c.k; e.k2 = c.k2; e.d_is_f32 = c.d_is_f32;
    cudaEventRecord(e.e0, stream);
    const int32_t s = gemm_nt_run_inner(c, stream);
    cudaEventRecord(e.e1, stream);
    g_prof.push_back(e);
    return s;
}

static int32_t gemm_nt_run_inner(const GemmCall& c, cudaStream_t stream) {
    // CTA-pair kernel first (256 x 256 cluster tiles); MFT_GEMM_2CTA=0 selects the single-CTA kernel everywhere
    static const int use_pair = [] { const char* e = std::getenv("MFT_GEMM_2CTA"); return e ? std::atoi(e) : 1; }();
    if (use_pair && device_status_word()) {
        const int32_t s2 = gemm_nt_run_2cta(c, stream);
        if (s2 != MFT_ERR_UNSUPPORTED) return s2;
    }
    if (c.epi == EPI_GLU_FWD || c.epi == EPI_GLU_BWD) return MFT_ERR_UNSUPPORTED;     // CTA-pair kernel only: the caller runs the unfused pair
    MFT_CHECK_ARG(c.a && c.b && c.m > 0 && c.n > 0 && c.k > 0, "gemm_nt: bad argument");
    MFT_CHECK_ARG(c.m < (1ll << 31) && c.n < (1ll << 31) && c.k < (1ll << 31), "gemm_nt: dimension too large");
    MFT_CHECK_ARG(c.epi == EPI_CE_STATS || c.d, "gemm_nt: null output");
    MFT_CHECK_ARG(!c.accumulate || c.d_is_f32, "gemm_nt: accumulate needs f32 D");
    MFT_CHECK_ARG(c.k2 >= 0 && c.k2 <= GEMM_BK, "gemm_nt: k2 must be in [0, 64]");
    MFT_CHECK_ARG(c.k2 == 0 || (c.a2 && c.b2), "gemm_nt: second segment needs a2 and b2");
    MFT_CHECK_ARG((c.epi == EPI_CE_STATS || c.ldd >= c.n) && c.lda >= c.k && c.ldb >= c.k, "gemm_nt: leading dimension too small");
    if (!device_status_word()) return fail(MFT_ERR_INVALID_ARG, "gemm_nt: call mft_init first");
    const int bn = c.epi == EPI_STORE ? pick_bn(c.n) : CE_TILE_N;
    CUtensorMap ma, mb, ma2, mb2;
    if (int32_t s = make_tmap_bf16(&ma, c.a, c.m, c.k, c.lda, GEMM_BM)) return s;
    if (int32_t s = make_tmap_bf16(&mb, c.b, c.n, c.k, c.ldb, bn)) return s;
    if (c.k2 > 0) {
        if (int32_t s = make_tmap_bf16(&ma2, c.a2, c.m, c.k2, c.lda2, GEMM_BM)) return s;
        if (int32_t s = make_tmap_bf16(&mb2, c.b2, c.n, c.k2, c.ldb2, bn)) return s;
    } else {
        ma2 = ma; mb2 = mb;
    }
    // bf16 outputs go through shared memory and TMA tensor stores (coalesced 128-byte rows, edges clipped by the
    // tensor map); f32 / accumulating outputs and oddly strided D keep the direct register -> global path
    CUtensorMap md = ma;
    const bool f32_tma = c.epi == EPI_STORE && c.d_is_f32 && (c.ldd % 4 == 0) && (reinterpret_cast<uintptr_t>(c.d) % 16 == 0);
    const bool tma_store = f32_tma || (c.epi != EPI_CE_STATS && !c.d_is_f32 && (c.ldd % 8 == 0) && (reinterpret_cast<uintptr_t>(c.d) % 16 == 0));
    if (f32_tma) {
        if (int32_t s = make_tmap_f32_out(&md, c.d, c.m, c.n, c.ldd)) return s;
    } else if (tma_store) {
        if (int32_t s = make_tmap_bf16(&md, c.d, c.m, c.n, c.ldd, 32)) return s;
    }
    MFT_CHECK_ARG(c.splits >= 0 && c.splits <= 64, "gemm_nt: bad K split");
    const bool can_split = f32_tma && c.k2 == 0;
    MFT_CHECK_ARG(c.splits <= 1 || can_split, "gemm_nt: a K split needs an aligned f32 output and no second segment");
    const int splits = (c.splits == 0 && !can_split) ? 1 : c.splits;
    GemmParams p{};
    p.m = (int)c.m; p.n = (int)c.n; p.k = (int)c.k; p.k2 = (int)c.k2;
    p.alpha = c.alpha; p.bias = c.bias; p.d = c.d; p.ldd = c.ldd;
    p.d_is_f32 = c.d_is_f32; p.accumulate = c.accumulate; p.tma_store = tma_store ? 1 : 0;
    p.f32_reduce = (f32_tma && c.accumulate) ? 1 : 0; p.splits = splits;
    p.status = device_status_word();
    p.ce_tgt = c.ce_tgt; p.ce_lse = c.ce_lse; p.ce_nvalid = c.ce_nvalid; p.ce_nvalid_override = c.ce_nvalid_override;
    p.ce_dloss = c.ce_dloss; p.ce_col_offset = c.ce_col_offset; p.ce_partials = c.ce_partials;
    p.ce_partial_ld = c.ce_partial_ld; p.ce_tgt_logit = c.ce_tgt_logit; p.ce_flag = c.ce_flag;
    if (c.epi == EPI_CE_STATS) return launch_gemm<CE_TILE_N, EPI_CE_STATS>(ma, mb, ma2, mb2, md, p, stream);
    if (c.epi == EPI_CE_GRAD) return launch_gemm<CE_TILE_N, EPI_CE_GRAD>(ma, mb, ma2, mb2, md, p, stream);
    if (c.epi == EPI_CE_P) {
        if (!tma_store) return fail(MFT_ERR_INVALID_ARG, "gemm_nt: the softmax-numerator epilogue needs an aligned bf16 output");
        return launch_gemm<CE_TILE_N, EPI_CE_P>(ma, mb, ma2, mb2, md, p, stream);
    }
    if (bn == 256) return launch_gemm<256, EPI_STORE>(ma, mb, ma2, mb2, md, p, stream);
    if (bn == 192) return launch_gemm<192, EPI_STORE>(ma, mb, ma2, mb2, md, p, stream);
    if (bn == 128) return launch_gemm<128, EPI_STORE>(ma, mb, ma2, mb2, md, p, stream);
    return launch_gemm<64, EPI_STORE>(ma, mb, ma2, mb2, md, p, stream);
}

}  // namespace mft

using namespace mft;

extern "C" int32_t mft_profile_gemm(int32_t enable) {
    for (auto& e : g_prof) { cudaEventDestroy(e.e0); cudaEventDestroy(e.e1); }
    g_prof.clear();
    g_prof_on = enable != 0;
    return MFT_OK;
}

extern "C" int32_t mft_profile_gemm_report_epi(int32_t epilogue_mask, double* flops, double* ms, int64_t* launches) {
    MFT_CHECK_ARG(flops && ms && launches, "mft_profile_gemm_report: null pointer");
    double f = 0, t = 0;
    int64_t n = 0;
    for (auto& e : g_prof) {
        if (!((epilogue_mask >> e.epi) & 1)) continue;
        if (int32_t s = check_cuda(cudaEventSynchronize(e.e1), "profile sync")) return s;
        float dt = 0.f;
        cudaEventElapsedTime(&dt, e.e0, e.e1);
        f += e.flops; t += dt; ++n;
    }
    *flops = f; *ms = t; *launches = n;
    return MFT_OK;
}

extern "C" int32_t mft_profile_gemm_launch(int64_t index, int64_t* shape_mnk_k2, int32_t* epilogue, int32_t* d_is_f32, double* ms) {
    MFT_CHECK_ARG(shape_mnk_k2 && epilogue && d_is_f32 && ms, "mft_profile_gemm_launch: null pointer");
    MFT_CHECK_ARG(index >= 0 && index < (int64_t)g_prof.size(), "mft_profile_gemm_launch: index beyond the recorded launches");
    const ProfEntry& e = g_prof[(size_t)index];
    if (int32_t s = check_cuda(cudaEventSynchronize(e.e1), "profile sync")) return s;
    float dt = 0.f;
    cudaEventElapsedTime(&dt, e.e0, e.e1);
    shape_mnk_k2[0] = e.m; shape_mnk_k2[1] = e.n; shape_mnk_k2[2] = e.k; shape_mnk_k2[3] = e.k2;
    *epilogue = e.epi; *d_is_f32 = e.d_is_f32; *ms = dt;
    return MFT_OK;
}

extern "C" int32_t mft_profile_gemm_report(double* flops, double* ms, int64_t* launches) {
    return mft_profile_gemm_report_epi(~0, flops, ms, launches);
}

extern "C" int32_t mft_glu_linear_fwd(int32_t kind, const void* x, int64_t ldx, const void* w_nk, int64_t ldw, int64_t m, int64_t inter, int64_t k,
                                      const void* xa, int64_t ldxa, const void* b_nk, int64_t ldb2, int64_t k2, const float* bias,
                                      void* gu, int64_t ld_gu, void* act, int64_t ld_act, mft_stream_t stream) {
    MFT_CHECK_ARG(kind == MFT_ACT_GEGLU || kind == MFT_ACT_SWIGLU, "mft_glu_linear_fwd: kind must be MFT_ACT_GEGLU or MFT_ACT_SWIGLU");
    MFT_CHECK_ARG(x && w_nk && gu && act && m > 0 && inter > 0 && k > 0 && ld_gu >= 2 * inter && ld_act >= inter, "mft_glu_linear_fwd: bad argument");
    GemmCall c;
    c.a = x; c.lda = ldx; c.b = w_nk; c.ldb = ldw; c.m = m; c.n = 2 * inter; c.k = k;
    c.a2 = xa; c.lda2 = ldxa; c.b2 = b_nk; c.ldb2 = ldb2; c.k2 = k2;
    c.bias = bias; c.d = gu; c.ldd = ld_gu; c.epi = EPI_GLU_FWD;
    c.glu_geglu = kind == MFT_ACT_GEGLU; c.glu_inter = inter; c.aux = act; c.ld_aux = ld_act;
    return gemm_nt_run(c, as_stream(stream));
}

extern "C" int32_t mft_glu_linear_bwd(int32_t kind, const void* dy, int64_t lddy, const void* w_kn, int64_t ldw, int64_t m, int64_t inter, int64_t k,
                                      const void* a2, int64_t lda2, const void* b2, int64_t ldb2, int64_t k2,
                                      const void* gu, int64_t ld_gu, void* dgu, int64_t ld_dgu, mft_stream_t stream) {
    MFT_CHECK_ARG(kind == MFT_ACT_GEGLU || kind == MFT_ACT_SWIGLU, "mft_glu_linear_bwd: kind must be MFT_ACT_GEGLU or MFT_ACT_SWIGLU");
    MFT_CHECK_ARG(dy && w_kn && gu && dgu && m > 0 && inter > 0 && k > 0 && ld_gu >= 2 * inter && ld_dgu >= 2 * inter, "mft_glu_linear_bwd: bad argument");
    GemmCall c;
    c.a = dy; c.lda = lddy; c.b = w_kn; c.ldb = ldw; c.m = m; c.n = inter; c.k = k;
    c.a2 = a2; c.lda2 = lda2; c.b2 = b2; c.ldb2 = ldb2; c.k2 = k2;
    c.d = dgu; c.ldd = ld_dgu; c.epi = EPI_GLU_BWD;
    c.glu_geglu = kind == MFT_ACT_GEGLU; c.glu_inter = inter; c.aux = const_cast<void*>(gu); c.ld_aux = ld_gu;
    return gemm_nt_run(c, as_stream(stream));
}

extern "C" int32_t mft_gemm_nt_tile_cols(int64_t m, int64_t n, int64_t k, int64_t k2, int32_t d_dtype, int32_t* tile_cols_host) {
    MFT_CHECK_ARG(tile_cols_host && m > 0 && n > 0 && k > 0 && k2 >= 0, "mft_gemm_nt_tile_cols: bad argument");
    MFT_CHECK_ARG(d_dtype == MFT_F32 || d_dtype == MFT_BF16, "mft_gemm_nt_tile_cols: D must be f32 or bf16");
    *tile_cols_host = gemm_nt_pair_tile_cols(m, n, k, k2, d_dtype == MFT_F32);
    return MFT_OK;
}

extern "C" int32_t mft_gemm_nt(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k,
                               const void* a2, int64_t lda2, const void* b2, int64_t ldb2, int64_t k2, const float* bias,
                               float alpha, void* d, int64_t ldd, int32_t d_dtype, int32_t accumulate, mft_stream_t stream) {
    MFT_CHECK_ARG(d_dtype == MFT_F32 || d_dtype == MFT_BF16, "mft_gemm_nt: D must be f32 or bf16");
    GemmCall c;
    c.a = a; c.lda = lda; c.b = b; c.ldb = ldb; c.m = m; c.n = n; c.k = k;
    c.a2 = a2; c.lda2 = lda2; c.b2 = b2; c.ldb2 = ldb2; c.k2 = k2;
    c.bias = bias; c.alpha = alpha; c.d = d; c.ldd = ldd; c.d_is_f32 = d_dtype == MFT_F32; c.accumulate = accumulate;
    c.splits = 0;     // f32 outputs: K is split when that fills the last wave of tiles better
    return gemm_nt_run(c, as_stream(stream));
}
