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
// Fused  : forward and backward in ONE sweep over the vocabulary (training step).  A first GEMM over panel 0
//           gives every row a reference value m_ref (the log-sum-exp of that panel, a lower bound of the full
//           one).  Then per panel GEMM 1 writes the un-normalised numerators P = exp(logit - m_ref) as bf16
//           and their per-row sums, GEMM 2 accumulates D += P x table[panel, :] in fp32, and a last kernel
//           forms lse = m_ref + log(sum P), the loss and dHidden = (D / sum P - table[label]) * dloss / n_valid.
//           The logits are computed once instead of twice.  A row whose logits exceed m_ref by more than the
//           trusted range is flagged by GEMM 1 and recomputed exactly on the CUDA cores.
// Semantics follow lm_cross_entropy of the reference: row (b, s) is scored
// against labels[b, s+1]; the last position of a sequence and labels equal to
// ignore_index contribute nothing; mean over scored rows; NaN if none.
#include "common.cuh"
#include "gemm_sm100.h"

namespace mft {
namespace {

constexpr int64_t PANEL = 8192;                         // granularity of a vocabulary panel, and the probe of the fused sweep
int64_t g_panel_budget = 12ll << 30;                    // bytes the bf16 [T, panel] buffer may take

inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct CeWorkspace {
    int32_t* tgt;
    float* tgt_logit;
    float2* partials;
    double* loss_sum;      // [1]
    int32_t* count;        // [1] scratch count for the backward
    __nv_bfloat16* g;      // [T, panel]
    float* dh_acc;         // [T, H]
    float* m_ref;          // [T] reference exponent of the fused sweep
    int32_t* row_flag;     // [T] rows the fused sweep must recompute exactly
    int64_t ntiles, panel, total;
};

CeWorkspace carve(void* base, int64_t T, int64_t H, int64_t V) {
    CeWorkspace w{};
    w.ntiles = (V + CE_TILE_N - 1) / CE_TILE_N;
    // as many PANEL-column blocks as the budget allows: one GEMM pair per panel, so fewer panels mean longer
    // K loops in the dHidden GEMM and fewer passes over its f32 accumulator
    const int64_t v_pad = (V + 255) / 256 * 256;
    const int64_t by_budget = std::max<int64_t>(1, g_panel_budget / (T * 2) / PANEL) * PANEL;
    w.panel = std::min(v_pad, by_budget);
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
    w.m_ref = reinterpret_cast<float*>(take(T * 4));
    w.row_flag = reinterpret_cast<int32_t*>(take(T * 4));
    w.total = off;
    return w;
}

__global__ void ce_prepare_kernel(const int32_t* __restrict__ labels, int64_t batch, int64_t seq, int64_t vocab,
                                  int ignore_index, int32_t* __restrict__ tgt, int32_t* __restrict__ n_valid,
                                  int32_t* __restrict__ status) {
    dep_trigger();
    dep_wait();
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

__global__ void ce_reduce_kernel(const float2* __restrict__ partials, int64_t ntiles, int64_t ld, const int32_t* __restrict__ tgt,
                                 const float* __restrict__ tgt_logit, float* __restrict__ lse, double* __restrict__ loss_sum,
                                 int64_t T) {
    dep_trigger();
    dep_wait();
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= T) return;
    float m = -INFINITY, s = 0.f;
    for (int64_t i = lane; i < ntiles; i += 32) {
        const float2 pr = partials[row * ld + i];
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
        if (loss_sum && tgt[row] >= 0) atomicAdd(loss_sum, (double)(l - tgt_logit[row]));
    }
}

__global__ void ce_finalize_kernel(const double* loss_sum, const int32_t* n_valid, float* loss) {
    dep_trigger();
    dep_wait();
    const int n = *n_valid;
    *loss = n > 0 ? (float)(*loss_sum / (double)n) : NAN;
}


// ---- fused sweep: last step for the rows GEMM 1 did not flag.  One block per row.
__global__ void ce_fused_finish_kernel(const float2* __restrict__ partials, int64_t ntiles, const int32_t* __restrict__ tgt,
                                       const float* __restrict__ tgt_logit, const float* __restrict__ m_ref,
                                       const int32_t* __restrict__ row_flag, const float* __restrict__ dacc,
                                       const __nv_bfloat16* __restrict__ table, int64_t H, const int32_t* __restrict__ n_valid,
                                       int64_t nv_override, float dloss, float* __restrict__ lse, double* __restrict__ loss_sum,
                                       __nv_bfloat16* __restrict__ dh) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    if (row_flag[row]) return;
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < ntiles; i += blockDim.x) s += partials[row * ntiles + i].y;
    s = block_sum(s, scratch);
    const int t = tgt[row];
    if (threadIdx.x == 0) {
        const float l = m_ref[row] + logf(s);
        lse[row] = l;
        if (t >= 0) atomicAdd(loss_sum, (double)(l - tgt_logit[row]));
    }
    const long long nv = nv_override > 0 ? nv_override : (long long)*n_valid;
    const float coef = (t >= 0 && nv > 0) ? dloss / (float)nv : 0.f;
    __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(dh + row * H);
    if (coef == 0.f) {
        for (int64_t i = threadIdx.x; i < H / 2; i += blockDim.x) out[i] = __floats2bfloat162_rn(0.f, 0.f);
        return;
    }
    const float inv = 1.f / s;
    const float2* d2 = reinterpret_cast<const float2*>(dacc + row * H);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(table + (int64_t)t * H);
    for (int64_t i = threadIdx.x; i < H / 2; i += blockDim.x) {
        const float2 d = d2[i];
        const float2 w = __bfloat1622float2(w2[i]);
        out[i] = __floats2bfloat162_rn((d.x * inv - w.x) * coef, (d.y * inv - w.y) * coef);
    }
}

// ---- fused sweep: exact recomputation of the flagged rows on the CUDA cores (two sweeps over the vocabulary
// per row; slow, and only ever run for rows whose logits left the range GEMM 1 trusts).
// Dynamic shared memory: hidden row [H] + one dHidden accumulator [H] per warp.
__global__ void ce_row_fixup_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ table,
                                    const int32_t* __restrict__ tgt, const int32_t* __restrict__ row_flag, int64_t T, int64_t H,
                                    int64_t V, const int32_t* __restrict__ n_valid, int64_t nv_override, float dloss,
                                    float* __restrict__ lse, double* __restrict__ loss_sum, __nv_bfloat16* __restrict__ dh) {
    dep_trigger();
    dep_wait();
    extern __shared__ float fix_smem[];
    __shared__ float red_m[32], red_s[32], tgt_l, row_lse;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* hrow = fix_smem;
    float* dw = fix_smem + H + (int64_t)warp * H;
    for (int64_t row = blockIdx.x; row < T; row += gridDim.x) {
        if (!row_flag[row]) continue;
        __syncthreads();
        for (int64_t i = threadIdx.x; i < H; i += blockDim.x) hrow[i] = __bfloat162float(hidden[row * H + i]);
        for (int64_t i = lane; i < H; i += 32) dw[i] = 0.f;
        __syncthreads();
        const int t = tgt[row];
        float m = -INFINITY, s = 0.f;
        for (int64_t j = warp; j < V; j += nwarps) {
            const __nv_bfloat16* wr = table + j * H;
            float dot = 0.f;
            for (int64_t i = lane; i < H; i += 32) dot += hrow[i] * __bfloat162float(wr[i]);
            dot = warp_sum(dot);
            if (j == t && lane == 0) tgt_l = dot;
            const float nm = fmaxf(m, dot);
            s = s * __expf(m - nm) + __expf(dot - nm);
            m = nm;
        }
        if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float mm = -INFINITY, ss = 0.f;
            for (int w = 0; w < nwarps; ++w) mm = fmaxf(mm, red_m[w]);
            for (int w = 0; w < nwarps; ++w) if (red_m[w] > -INFINITY) ss += red_s[w] * __expf(red_m[w] - mm);
            const float l = mm + logf(ss);
            row_lse = l;
            lse[row] = l;
            if (t >= 0) atomicAdd(loss_sum, (double)(l - tgt_l));
        }
        __syncthreads();
        const long long nv = nv_override > 0 ? nv_override : (long long)*n_valid;
        const float coef = (t >= 0 && nv > 0) ? dloss / (float)nv : 0.f;
        if (coef != 0.f) {
            const float l = row_lse;
            for (int64_t j = warp; j < V; j += nwarps) {
                const __nv_bfloat16* wr = table + j * H;
                float dot = 0.f;
                for (int64_t i = lane; i < H; i += 32) dot += hrow[i] * __bfloat162float(wr[i]);
                dot = warp_sum(dot);
                const float pj = __expf(dot - l) - (j == t ? 1.f : 0.f);
                for (int64_t i = lane; i < H; i += 32) dw[i] += pj * __bfloat162float(wr[i]);
            }
        }
        __syncthreads();
        for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
            float acc = 0.f;
            for (int w = 0; w < nwarps; ++w) acc += fix_smem[H + (int64_t)w * H + i];
            dh[row * H + i] = __float2bfloat16_rn(acc * coef);
        }
    }
}

// ---- dense-logits variants
__global__ void ce_dense_fwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ tgt, int64_t vocab,
                                    float* __restrict__ lse, double* __restrict__ loss_sum) {
    dep_trigger();
    dep_wait();
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
    dep_trigger();
    dep_wait();
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

extern "C" int64_t mft_lmhead_ce_set_panel_budget(int64_t bytes) {
    const int64_t old = g_panel_budget;
    if (bytes > 0) g_panel_budget = bytes;
    return old;
}

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
    launch_dep(ce_prepare_kernel, dim3((unsigned)std::min<int64_t>((T + 255) / 256, 1024)), dim3(256), (size_t)(0), st, labels, batch, seq, vocab, ignore_index, w.tgt, n_valid_dev, status_dev);
    MFT_LAUNCH_CHECK("ce_prepare");
    GemmCall c;
    c.a = hidden_bf16; c.lda = hidden; c.b = table_bf16; c.ldb = hidden; c.m = T; c.n = vocab; c.k = hidden;
    c.epi = EPI_CE_STATS; c.ce_tgt = w.tgt; c.ce_partials = w.partials; c.ce_partial_ld = (int)w.ntiles; c.ce_tgt_logit = w.tgt_logit;
    if (int32_t s = gemm_nt_run(c, st)) return s;
    launch_dep(ce_reduce_kernel, dim3((unsigned)((T * 32 + 255) / 256)), dim3(256), (size_t)(0), st, w.partials, w.ntiles, w.ntiles, w.tgt, w.tgt_logit, lse, w.loss_sum, T);
    MFT_LAUNCH_CHECK("ce_reduce");
    launch_dep(ce_finalize_kernel, dim3(1), dim3(1), (size_t)(0), st, w.loss_sum, n_valid_dev, loss_dev);
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
    launch_dep(ce_prepare_kernel, dim3((unsigned)std::min<int64_t>((T + 255) / 256, 1024)), dim3(256), (size_t)(0), st, labels, batch, seq, vocab, ignore_index, w.tgt, w.count, nullptr);
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


extern "C" int32_t mft_lmhead_ce_fused(const void* hidden_bf16, const void* table_bf16, const void* table_t_bf16, int64_t table_t_ld,
                                       const int32_t* labels, int64_t batch, int64_t seq, int64_t hidden, int64_t vocab,
                                       int32_t ignore_index, int64_t n_valid_override, float dloss, float* loss_dev,
                                       int32_t* n_valid_dev, float* lse, void* dhidden_bf16, int32_t* status_dev, void* workspace,
                                       int64_t workspace_bytes, mft_stream_t stream) {
    MFT_CHECK_ARG(hidden_bf16 && table_bf16 && table_t_bf16 && labels && loss_dev && n_valid_dev && lse && dhidden_bf16 && workspace,
                  "mft_lmhead_ce_fused: null pointer");
    MFT_CHECK_ARG(batch > 0 && seq > 0 && hidden > 0 && vocab > 0 && hidden % 8 == 0 && table_t_ld >= vocab && table_t_ld % 8 == 0,
                  "mft_lmhead_ce_fused: bad size");
    const int64_t T = batch * seq, H = hidden;
    CeWorkspace w = carve(workspace, T, H, vocab);
    MFT_CHECK_ARG(workspace_bytes >= w.total, "mft_lmhead_ce_fused: workspace too small");
    constexpr int FIX_THREADS = 256;
    const size_t fix_smem = (size_t)(1 + FIX_THREADS / 32) * H * sizeof(float);
    MFT_CHECK_ARG(fix_smem <= 200 * 1024, "mft_lmhead_ce_fused: hidden size too large");
    cudaStream_t st = as_stream(stream);
    if (int32_t s = check_cuda(cudaMemsetAsync(n_valid_dev, 0, 4, st), "ce memset")) return s;
    if (int32_t s = check_cuda(cudaMemsetAsync(w.loss_sum, 0, 8, st), "ce memset")) return s;
    if (int32_t s = check_cuda(cudaMemsetAsync(w.row_flag, 0, (size_t)T * 4, st), "ce memset")) return s;
    launch_dep(ce_prepare_kernel, dim3((unsigned)std::min<int64_t>((T + 255) / 256, 1024)), dim3(256), (size_t)(0), st, labels, batch, seq, vocab, ignore_index, w.tgt, n_valid_dev, status_dev);
    MFT_LAUNCH_CHECK("ce_prepare");
    // reference exponent per row: log-sum-exp of panel 0
    {
        const int64_t vc = std::min(PANEL, vocab);
        GemmCall c;
        c.a = hidden_bf16; c.lda = H; c.b = table_bf16; c.ldb = H; c.m = T; c.n = vc; c.k = H;
        c.epi = EPI_CE_STATS; c.ce_tgt = w.tgt; c.ce_partials = w.partials; c.ce_partial_ld = (int)w.ntiles; c.ce_tgt_logit = w.tgt_logit;
        if (int32_t s = gemm_nt_run(c, st)) return s;
        launch_dep(ce_reduce_kernel, dim3((unsigned)((T * 32 + 255) / 256)), dim3(256), (size_t)(0), st, w.partials, (vc + CE_TILE_N - 1) / CE_TILE_N, w.ntiles, w.tgt,
                                                                         w.tgt_logit, w.m_ref, nullptr, T);
        MFT_LAUNCH_CHECK("ce_reduce");
    }
    for (int64_t v0 = 0; v0 < vocab; v0 += w.panel) {
        const int64_t vc = std::min(w.panel, vocab - v0);
        GemmCall c;
        c.a = hidden_bf16; c.lda = H;
        c.b = static_cast<const __nv_bfloat16*>(table_bf16) + v0 * H; c.ldb = H;
        c.m = T; c.n = vc; c.k = H;
        c.d = w.g; c.ldd = w.panel; c.d_is_f32 = 0;
        c.epi = EPI_CE_P; c.ce_tgt = w.tgt; c.ce_lse = w.m_ref; c.ce_col_offset = (int)v0;
        c.ce_partials = w.partials; c.ce_partial_ld = (int)w.ntiles; c.ce_tgt_logit = w.tgt_logit; c.ce_flag = w.row_flag;
        if (int32_t s = gemm_nt_run(c, st)) return s;
        GemmCall d;
        d.a = w.g; d.lda = w.panel;
        d.b = static_cast<const __nv_bfloat16*>(table_t_bf16) + v0; d.ldb = table_t_ld;
        d.m = T; d.n = H; d.k = vc;
        d.d = w.dh_acc; d.ldd = H; d.d_is_f32 = 1; d.accumulate = v0 > 0; d.splits = 0;
        if (int32_t s = gemm_nt_run(d, st)) return s;
    }
    launch_dep(ce_fused_finish_kernel, dim3((unsigned)T), dim3(128), (size_t)(0), st, w.partials, w.ntiles, w.tgt, w.tgt_logit, w.m_ref, w.row_flag, w.dh_acc,
                                                       static_cast<const __nv_bfloat16*>(table_bf16), H, n_valid_dev, n_valid_override,
                                                       dloss, lse, w.loss_sum, static_cast<__nv_bfloat16*>(dhidden_bf16));
    MFT_LAUNCH_CHECK("ce_fused_finish");
    static bool fix_attr = false;
    if (!fix_attr) {
        if (int32_t s = check_cuda(cudaFuncSetAttribute(ce_row_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "ce fixup attribute")) return s;
        fix_attr = true;
    }
    launch_dep(ce_row_fixup_kernel, dim3((unsigned)std::min<int64_t>(T, 148 * 4)), dim3(FIX_THREADS), (size_t)(fix_smem), st, 
        static_cast<const __nv_bfloat16*>(hidden_bf16), static_cast<const __nv_bfloat16*>(table_bf16), w.tgt, w.row_flag, T, H, vocab,
        n_valid_dev, n_valid_override, dloss, lse, w.loss_sum, static_cast<__nv_bfloat16*>(dhidden_bf16));
    MFT_LAUNCH_CHECK("ce_row_fixup");
    launch_dep(ce_finalize_kernel, dim3(1), dim3(1), (size_t)(0), st, w.loss_sum, n_valid_dev, loss_dev);
    MFT_LAUNCH_CHECK("ce_finalize");
    return MFT_OK;
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
    launch_dep(ce_prepare_kernel, dim3((unsigned)std::min<int64_t>((T + 255) / 256, 1024)), dim3(256), (size_t)(0), st, labels, batch, seq, vocab, ignore_index, tgt_scratch, n_valid_dev, status_dev);
    MFT_LAUNCH_CHECK("ce_prepare");
    launch_dep(ce_dense_fwd_kernel, dim3((unsigned)T), dim3(256), (size_t)(0), st, logits, tgt_scratch, vocab, lse, loss_scratch);
    MFT_LAUNCH_CHECK("ce_dense_fwd");
    launch_dep(ce_finalize_kernel, dim3(1), dim3(1), (size_t)(0), st, loss_scratch, n_valid_dev, loss_dev);
    MFT_LAUNCH_CHECK("ce_finalize");
    return MFT_OK;
}

extern "C" int32_t mft_ce_dense_bwd(const float* logits, const int32_t* tgt_scratch, int64_t batch, int64_t seq, int64_t vocab,
                                    const float* lse, const int32_t* n_valid_dev, float dloss, float* dlogits,
                                    mft_stream_t stream) {
    MFT_CHECK_ARG(logits && tgt_scratch && lse && n_valid_dev && dlogits && batch > 0 && seq > 0 && vocab > 0, "mft_ce_dense_bwd: bad argument");
    launch_dep(ce_dense_bwd_kernel, dim3((unsigned)(batch * seq)), dim3(256), (size_t)(0), as_stream(stream), logits, tgt_scratch, vocab, lse, n_valid_dev, dloss, dlogits);
    MFT_LAUNCH_CHECK("ce_dense_bwd");
    return MFT_OK;
}
