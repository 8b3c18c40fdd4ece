// lm head + shifted cross-entropy without materialising the [T, V] logits.
//
// Forward : one tcgen05 GEMM hidden[T,H] x table[V,H]^T whose epilogue reduces
//           every 128 x 256 logit tile to per-row (max, sum exp) partials and
//           picks the label logit; a small kernel merges the partials into the
//           row log-sum-exp and the mean loss.
// Backward: the vocabulary is cut into panels of PANEL columns.  Per panel the
//           logits are recomputed by the same GEMM with an epilogue that writes
//           G = (softmax - onehot) * dloss / n_valid as bf16 [T, PANEL], and a
//           second GEMM accumulates dHidden += G x table[panel, :] in fp32.
// Semantics follow lm_cross_entropy of the reference: row (b, s) is scored
// against labels[b, s+1]; the last position of a sequence and labels equal to
// ignore_index contribute nothing; mean over scored rows; NaN if none.
#include "common.cuh"
#include "gemm_sm100.h"

namespace mft {
namespace {

constexpr int64_t PANEL = 8192;

inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct CeWorkspace {
    int32_t* tgt;
    float* tgt_logit;
    float2* partials;
    double* loss_sum;      // [1]
    int32_t* count;        // [1] scratch count for the backward
    __nv_bfloat16* g;      // [T, panel]
    float* dh_acc;         // [T, H]
    int64_t ntiles, panel, total;
};

CeWorkspace carve(void* base, int64_t T, int64_t H, int64_t V) {
    CeWorkspace w{};
    w.ntiles = (V + CE_TILE_N - 1) / CE_TILE_N;
    w.panel = V < PANEL ? (V + 255) / 256 * 256 : PANEL;
    uint8_t* p = static_cast<uint8_t*>(base);
    int64_t off = 0;
    auto take = [&](int64_t bytes) { uint8_t* r = p ? p + off : nullptr; off += align256(bytes); return r; };
    w.tgt = reinterpret_cast<int32_t*>(take(T * 4));
    w.tgt_logit = reinterpret_cast<float*>(take(T * 4));
    w.partials = reinterpret_cast<float2*>(take(T * w.ntiles * 8));
    w.loss_sum = reinterpret_cast<double*>(take(8));
    w.count = reinterpret_cast<int32_t*>(take(4));
    w.g = reinterpret_cast<__nv_bfloat16*>(take(T * w.panel * 2));
    w.dh_acc = reinterpret_cast<float*>(take(T * H * 4));
    w.total = off;
    return w;
}

__global__ void ce_prepare_kernel(const int32_t* __restrict__ labels, int64_t batch, int64_t seq, int64_t vocab,
                                  int ignore_index, int32_t* __restrict__ tgt, int32_t* __restrict__ n_valid,
                                  int32_t* __restrict__ status) {
    __shared__ float scratch[32];
    const int64_t total = batch * seq;
    int local = 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t s = t % seq;
        int32_t out = -1;
        if (s + 1 < seq) {
            const int32_t lab = labels[t + 1];
            if (lab != ignore_index) {
                if (lab < 0 || lab >= vocab) { if (status) atomicExch(status, MFT_ERR_BOUNDS); }
                else { out = lab; ++local; }
            }
        }
        tgt[t] = out;
    }
    const float tot = block_sum((float)local, scratch);   // exact: block counts stay far below 2^24
    if (threadIdx.x == 0 && tot > 0.f) atomicAdd(n_valid, (int32_t)tot);
}

__global__ void ce_reduce_kernel(const float2* __restrict__ partials, int64_t ntiles, const int32_t* __restrict__ tgt,
                                 const float* __restrict__ tgt_logit, float* __restrict__ lse, double* __restrict__ loss_sum,
                                 int64_t T) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= T) return;
    float m = -INFINITY, s = 0.f;
    for (int64_t i = lane; i < ntiles; i += 32) {
        const float2 pr = partials[row * ntiles + i];
        const float nm = fmaxf(m, pr.x);
        s = s * __expf(m - nm) + pr.y * __expf(pr.x - nm);
        m = nm;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
        const float nm = fmaxf(m, om);
        s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
        m = nm;
    }
    if (lane == 0) {
        const float l = m + logf(s);
        lse[row] = l;
        if (tgt[row] >= 0) atomicAdd(loss_sum, (double)(l - tgt_logit[row]));
    }
}

__global__ void ce_finalize_kernel(const double* loss_sum, const int32_t* n_valid, float* loss) {
    const int n = *n_valid;
    *loss = n > 0 ? (float)(*loss_sum / (double)n) : NAN;
}

// ---- dense-logits variants
__global__ void ce_dense_fwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ tgt, int64_t vocab,
                                    float* __restrict__ lse, double* __restrict__ loss_sum) {
    __shared__ float scratch[32];
    __shared__ float bmax;
    const int64_t row = blockIdx.x;
    const float* lr = logits + row * vocab;
    float m = -INFINITY;
    for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, lr[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = -INFINITY;
        for (int i = 0; i < (blockDim.x + 31) / 32; ++i) mm = fmaxf(mm, scratch[i]);
        bmax = mm;
    }
    __syncthreads();
    m = bmax;
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(lr[i] - m);
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) {
        const float l = m + logf(s);
        lse[row] = l;
        if (tgt[row] >= 0) atomicAdd(loss_sum, (double)(l - lr[tgt[row]]));
    }
}
__global__ void ce_dense_bwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ tgt, int64_t vocab,
                                    const float* __restrict__ lse, const int32_t* __restrict__ n_valid, float dloss,
                                    float* __restrict__ dlogits) {
    const int64_t row = blockIdx.x;
    const int t = tgt[row];
    const int n = *n_valid;
    const float coef = (t >= 0 && n > 0) ? dloss / (float)n : 0.f;
    const float l = lse[row];
    for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float pr = expf(logits[row * vocab + i] - l);
        dlogits[row * vocab + i] = coef == 0.f ? 0.f : (pr - (i == t ? 1.f : 0.f)) * coef;
    }
}

}  // namespace
}  // namespace mft

using namespace mft;

extern "C" int64_t mft_lmhead_ce_workspace_bytes(int64_t n_tokens, int64_t hidden, int64_t vocab) {
    if (n_tokens <= 0 || hidden <= 0 || vocab <= 0) return 0;
    return carve(nullptr, n_tokens, hidden, vocab).total;
}

extern "C" int32_t mft_lmhead_ce_fwd(const void* hidden_bf16, const void* table_bf16, const int32_t* labels, int64_t batch,
                                     int64_t seq, int64_t hidden, int64_t vocab, int32_t ignore_index, float* loss_dev,
                                     int32_t* n_valid_dev, float* lse, int32_t* status_dev, void* workspace,
                                     int64_t workspace_bytes, mft_stream_t stream) {
    MFT_CHECK_ARG(hidden_bf16 && table_bf16 && labels && loss_dev && n_valid_dev && lse && workspace, "mft_lmhead_ce_fwd: null pointer");
    MFT_CHECK_ARG(batch > 0 && seq > 0 && hidden > 0 && vocab > 0, "mft_lmhead_ce_fwd: bad size");
    const int64_t T = batch * seq;
    CeWorkspace w = carve(workspace, T, hidden, vocab);
    MFT_CHECK_ARG(workspace_bytes >= w.total, "mft_lmhead_ce_fwd: workspace too small");
    cudaStream_t st = as_stream(stream);
    if (int32_t s = check_cuda(cudaMemsetAsync(n_valid_dev, 0, 4, st), "ce memset")) return s;
    if (int32_t s = check_cuda(cudaMemsetAsync(w.loss_sum, 0, 8, st), "ce memset")) return s;
    ce_prepare_kernel<<<(unsigned)std::min<int64_t>((T + 255) / 256, 1024), 256, 0, st>>>(labels, batch, seq, vocab, ignore_index, w.tgt, n_valid_dev, status_dev);
    MFT_LAUNCH_CHECK("ce_prepare");
    GemmCall c;
    c.a = hidden_bf16; c.lda = hidden; c.b = table_bf16; c.ldb = hidden; c.m = T; c.n = vocab; c.k = hidden;
    c.epi = EPI_CE_STATS; c.ce_tgt = w.tgt; c.ce_partials = w.partials; c.ce_partial_ld = (int)w.ntiles; c.ce_tgt_logit = w.tgt_logit;
    if (int32_t s = gemm_nt_run(c, st)) return s;
    ce_reduce_kernel<<<(unsigned)((T * 32 + 255) / 256), 256, 0, st>>>(w.partials, w.ntiles, w.tgt, w.tgt_logit, lse, w.loss_sum, T);
    MFT_LAUNCH_CHECK("ce_reduce");
    ce_finalize_kernel<<<1, 1, 0, st>>>(w.loss_sum, n_valid_dev, loss_dev);
    MFT_LAUNCH_CHECK("ce_finalize");
    return MFT_OK;
}

extern "C" int32_t mft_lmhead_ce_bwd(const void* hidden_bf16, const void* table_bf16, const void* table_t_bf16,
                                     int64_t table_t_ld, const int32_t* labels, int64_t batch, int64_t seq, int64_t hidden,
                                     int64_t vocab, int32_t ignore_index, const float* lse, const int32_t* n_valid_dev,
                                     int64_t n_valid_override, float dloss, void* dhidden_bf16, void* workspace,
                                     int64_t workspace_bytes, mft_stream_t stream) {
    MFT_CHECK_ARG(hidden_bf16 && table_bf16 && table_t_bf16 && labels && lse && n_valid_dev && dhidden_bf16 && workspace, "mft_lmhead_ce_bwd: null pointer");
    MFT_CHECK_ARG(batch > 0 && seq > 0 && hidden > 0 && vocab > 0 && table_t_ld >= vocab && table_t_ld % 8 == 0, "mft_lmhead_ce_bwd: bad size");
    const int64_t T = batch * seq;
    CeWorkspace w = carve(workspace, T, hidden, vocab);
    MFT_CHECK_ARG(workspace_bytes >= w.total, "mft_lmhead_ce_bwd: workspace too small");
    cudaStream_t st = as_stream(stream);
    if (int32_t s = check_cuda(cudaMemsetAsync(w.count, 0, 4, st), "ce memset")) return s;
    ce_prepare_kernel<<<(unsigned)std::min<int64_t>((T + 255) / 256, 1024), 256, 0, st>>>(labels, batch, seq, vocab, ignore_index, w.tgt, w.count, nullptr);
    MFT_LAUNCH_CHECK("ce_prepare");
    for (int64_t v0 = 0; v0 < vocab; v0 += w.panel) {
        const int64_t vc = std::min(w.panel, vocab - v0);
        GemmCall c;
        c.a = hidden_bf16; c.lda = hidden;
        c.b = static_cast<const __nv_bfloat16*>(table_bf16) + v0 * hidden; c.ldb = hidden;
        c.m = T; c.n = vc; c.k = hidden;
        c.d = w.g; c.ldd = w.panel; c.d_is_f32 = 0;
        c.epi = EPI_CE_GRAD; c.ce_tgt = w.tgt; c.ce_lse = lse; c.ce_nvalid = n_valid_dev; c.ce_nvalid_override = n_valid_override;
        c.ce_dloss = dloss; c.ce_col_offset = (int)v0;
        if (int32_t s = gemm_nt_run(c, st)) return s;
        GemmCall d;
        d.a = w.g; d.lda = w.panel;
        d.b = static_cast<const __nv_bfloat16*>(table_t_bf16) + v0; d.ldb = table_t_ld;
        d.m = T; d.n = hidden; d.k = vc;
        d.d = w.dh_acc; d.ldd = hidden; d.d_is_f32 = 1; d.accumulate = v0 > 0;
        if (int32_t s = gemm_nt_run(d, st)) return s;
    }
    return mft_cast_f32_to_bf16(w.dh_acc, dhidden_bf16, T * hidden, stream);
}

extern "C" int32_t mft_ce_dense_fwd(const float* logits, const int32_t* labels, int64_t batch, int64_t seq, int64_t vocab,
                                    int32_t ignore_index, float* loss_dev, int32_t* n_valid_dev, float* lse, int32_t* tgt_scratch,
                                    double* loss_scratch, int32_t* status_dev, mft_stream_t stream) {
    MFT_CHECK_ARG(logits && labels && loss_dev && n_valid_dev && lse && tgt_scratch && loss_scratch, "mft_ce_dense_fwd: null pointer");
    MFT_CHECK_ARG(batch > 0 && seq > 0 && vocab > 0, "mft_ce_dense_fwd: bad size");
    const int64_t T = batch * seq;
    cudaStream_t st = as_stream(stream);
    if (int32_t s = check_cuda(cudaMemsetAsync(n_valid_dev, 0, 4, st), "ce memset")) return s;
    if (int32_t s = check_cuda(cudaMemsetAsync(loss_scratch, 0, 8, st), "ce memset")) return s;
    ce_prepare_kernel<<<(unsigned)std::min<int64_t>((T + 255) / 256, 1024), 256, 0, st>>>(labels, batch, seq, vocab, ignore_index, tgt_scratch, n_valid_dev, status_dev);
    MFT_LAUNCH_CHECK("ce_prepare");
    ce_dense_fwd_kernel<<<(unsigned)T, 256, 0, st>>>(logits, tgt_scratch, vocab, lse, loss_scratch);
    MFT_LAUNCH_CHECK("ce_dense_fwd");
    ce_finalize_kernel<<<1, 1, 0, st>>>(loss_scratch, n_valid_dev, loss_dev);
    MFT_LAUNCH_CHECK("ce_finalize");
    return MFT_OK;
}

extern "C" int32_t mft_ce_dense_bwd(const float* logits, const int32_t* tgt_scratch, int64_t batch, int64_t seq, int64_t vocab,
                                    const float* lse, const int32_t* n_valid_dev, float dloss, float* dlogits,
                                    mft_stream_t stream) {
    MFT_CHECK_ARG(logits && tgt_scratch && lse && n_valid_dev && dlogits && batch > 0 && seq > 0 && vocab > 0, "mft_ce_dense_bwd: bad argument");
    ce_dense_bwd_kernel<<<(unsigned)(batch * seq), 256, 0, as_stream(stream)>>>(logits, tgt_scratch, vocab, lse, n_valid_dev, dloss, dlogits);
    MFT_LAUNCH_CHECK("ce_dense_bwd");
    return MFT_OK;
}
