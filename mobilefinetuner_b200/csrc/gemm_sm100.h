// Internal interface of the tcgen05 NT GEMM: the C ABI entry point mft_gemm_nt
// and the lm-head cross-entropy routines both go through gemm_nt_run.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mft {

constexpr int EPI_STORE = 0;     // D = alpha*acc + bias (+ D)
constexpr int EPI_CE_STATS = 1;  // per-row (max, sum exp) over each 256-column tile; nothing stored
constexpr int EPI_CE_GRAD = 2;   // D(bf16) = (exp(acc - lse[row]) - [col == label[row]]) * dloss / n_valid
constexpr int EPI_CE_P = 3;      // D(bf16) = exp(acc - m_ref[row]); per-row sums of the stored values; label logit; overflow flag
// Gated MLP fused into the epilogue (CTA-pair kernel only).  The frozen gate|up weight is [2*inter, K]: gate rows first.
constexpr int EPI_GLU_FWD = 4;   // a pair tile = 128 gate columns + the 128 matching up columns; D gets gate|up, `aux` gets f(gate)*up
constexpr int EPI_GLU_BWD = 5;   // acc = d(act) tile of [M, inter]; reads gate|up from `aux`, D gets d_gate|d_up; d(act) is not stored
constexpr int CE_TILE_N = 256;   // column tile of the CE epilogues (fixes the layout of the partials)

struct GemmCall {
    const void* a = nullptr; int64_t lda = 0;
    const void* b = nullptr; int64_t ldb = 0;
    int64_t m = 0, n = 0, k = 0;
    const void* a2 = nullptr; int64_t lda2 = 0;
    const void* b2 = nullptr; int64_t ldb2 = 0;
    int64_t k2 = 0;
    const float* bias = nullptr;
    float alpha = 1.0f;
    void* d = nullptr; int64_t ldd = 0;
    int d_is_f32 = 0;
    int accumulate = 0;
    int splits = 1;               // f32 D only: cut K into this many ranges whose partial tiles are added in memory (0 = choose)
    int epi = EPI_STORE;
    const int32_t* ce_tgt = nullptr;
    const float* ce_lse = nullptr;
    const int32_t* ce_nvalid = nullptr;
    long long ce_nvalid_override = 0;
    float ce_dloss = 1.0f;
    int ce_col_offset = 0;
    float2* ce_partials = nullptr;
    int ce_partial_ld = 0;
    float* ce_tgt_logit = nullptr;
    int32_t* ce_flag = nullptr;
    // EPI_GLU_*: glu_geglu != 0 -> gelu(tanh) gating, else silu; inter = width of one half; aux = act out (FWD) / saved gate|up (BWD)
    int glu_geglu = 0;
    int64_t glu_inter = 0;
    void* aux = nullptr; int64_t ld_aux = 0;
};

// Kernel-side parameter block (by value in the launch).
struct GemmParams {
    int m, n, k, k2;
    int num_m_tiles, num_n_tiles;
    float alpha;
    const float* bias;
    void* d;
    long long ldd;
    int d_is_f32;
    int accumulate;
    int tma_store;                // D written through shared memory + TMA tensor stores (bf16) / stores or reductions (f32)
    int f32_reduce;               // f32 D through TMA: add into memory (accumulate, or K split) instead of overwrite
    int splits, kb_per_split, tiles_mn;   // K split: tile index = split * tiles_mn + (m, n) tile
    int32_t* status;
    // cross-entropy epilogues (lm head): see lmhead_ce.cu
    const int32_t* ce_tgt;        // [m] shifted label per row, -1 = row not scored
    const float* ce_lse;          // [m] row log-sum-exp (GRAD mode)
    const int32_t* ce_nvalid;     // device count of scored rows (GRAD mode)
    long long ce_nvalid_override; // > 0: use instead of *ce_nvalid
    float ce_dloss;
    int ce_col_offset;            // vocabulary index of column 0 of this GEMM
    float2* ce_partials;          // [m, ce_partial_ld] (max, sum exp) per row and column tile (STATS mode)
    int ce_partial_ld;
    float* ce_tgt_logit;          // [m] logit of the label column (STATS / P modes)
    int32_t* ce_flag;             // [m] set to 1 for a row whose exp(acc - m_ref) leaves the trusted range (P mode)
    int glu_geglu, glu_inter;     // EPI_GLU_*
};

// Tile order: groups of RASTER_GROUP column tiles, row tiles within a group, columns fastest.  CTAs that run at
// the same time then share a few A row-panels and a few B column-panels (instead of one B panel and every A panel),
// which keeps both operands L2-resident when M*K or N*K exceeds the L2.
constexpr int RASTER_GROUP = 8;
__host__ __device__ inline int tile_group_width(int tile, const GemmParams& p) {
    const int g = tile / (RASTER_GROUP * p.num_m_tiles);
    const int rest = p.num_n_tiles - g * RASTER_GROUP;
    return rest < RASTER_GROUP ? rest : RASTER_GROUP;
}
__host__ __device__ inline int tile_m(int tile, const GemmParams& p) {
    return (tile % (RASTER_GROUP * p.num_m_tiles)) / tile_group_width(tile, p);
}
__host__ __device__ inline int tile_n(int tile, const GemmParams& p) {
    return (tile / (RASTER_GROUP * p.num_m_tiles)) * RASTER_GROUP + (tile % (RASTER_GROUP * p.num_m_tiles)) % tile_group_width(tile, p);
}

int32_t gemm_nt_run(const GemmCall& c, cudaStream_t stream);
// CTA-pair (cta_group::2) variant for 256 x 256 cluster tiles; returns MFT_ERR_UNSUPPORTED when the call does not qualify.
int32_t gemm_nt_run_2cta(const GemmCall& c, cudaStream_t stream);
// columns of the pair kernel's tile for a plain-store call of this shape: 256, 384 (long K under a width that is a
// multiple of 384), or 0 when the pair kernel does not take the call
int gemm_nt_pair_tile_cols(int64_t m, int64_t n, int64_t k, int64_t k2, bool d_is_f32);
int32_t make_tmap_bf16(struct CUtensorMap_st* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
int32_t make_tmap_f32_out(struct CUtensorMap_st* map, const void* base, int64_t rows, int64_t cols, int64_t ld);
int num_sms();
bool gemm_profiling_enabled();       // per-launch event timing is on (incompatible with stream capture)

}  // namespace mft
