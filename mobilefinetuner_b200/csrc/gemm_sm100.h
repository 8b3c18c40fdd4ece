// Internal interface of the tcgen05 NT GEMM: the C ABI entry point mft_gemm_nt
// and the lm-head cross-entropy routines both go through gemm_nt_run.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mft {

constexpr int EPI_STORE = 0;     // D = alpha*acc + bias (+ D)
constexpr int EPI_CE_STATS = 1;  // per-row (max, sum exp) over each 256-column tile; nothing stored
constexpr int EPI_CE_GRAD = 2;   // D(bf16) = (exp(acc - lse[row]) - [col == label[row]]) * dloss / n_valid
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
};

int32_t gemm_nt_run(const GemmCall& c, cudaStream_t stream);
int num_sms();

}  // namespace mft
