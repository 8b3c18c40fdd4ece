// Causal / sliding-window grouped-query attention for head sizes the tiled kernels do not cover (anything other
// than 64, 128, 256: the few-wide heads of test-sized models).  Same arithmetic as the chain
// repeat_kv_heads -> matmul -> scale -> mask -> softmax -> matmul of the reference (graph/gemma_model.cpp:487-505,
// SoftmaxBackward core/backward_functions.cpp:306-349): scores and probabilities in f32, masks as index predicates,
// KV heads shared by index.  One CTA per query row (forward, dQ) or per key row (dK / dV); every load is a scalar
// bf16 load, so no stride or alignment condition applies.  Written for correctness on small shapes, not for speed.
#include "attention.h"

namespace mft {
namespace {

constexpr int GEN_THREADS = 128;

__device__ __forceinline__ int first_visible(int i, int window) { return window > 0 ? max(0, i - window + 1) : 0; }
__device__ __forceinline__ const __nv_bfloat16* row_ptr(const __nv_bfloat16* base, const mft_strides_t& s, int b, int t, int h) {
    return base + (int64_t)b * s.stride_b + (int64_t)t * s.stride_s + (int64_t)h * s.stride_h;
}
__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = lane < GEN_THREADS / 32 ? scratch[lane] : (is_max ? -INFINITY : 0.0f);
    return is_max ? warp_max(r) : warp_sum(r);
}

// smem: q row [hd] + probabilities [seq]
__global__ void __launch_bounds__(GEN_THREADS) attn_generic_fwd_kernel(AttnParams p, int hd) {
    dep_wait();
    extern __shared__ float sm[];
    __shared__ float red[32];
    float* qs = sm;
    float* ps = sm + hd;
    const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, kvh = h / p.rep;
    const __nv_bfloat16* q = row_ptr(p.q, p.sq, b, i, h);
    for (int d = threadIdx.x; d < hd; d += GEN_THREADS) qs[d] = bf16_to_f32(q[d]) * p.scale;
    __syncthreads();
    const int j0 = first_visible(i, p.window);
    float mx = -INFINITY;
    for (int j = j0 + threadIdx.x; j <= i; j += GEN_THREADS) {
        const __nv_bfloat16* k = row_ptr(p.k, p.sk, b, j, kvh);
        float s = 0.f;
        for (int d = 0; d < hd; ++d) s += qs[d] * bf16_to_f32(k[d]);
        ps[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);
    float sum = 0.f;
    for (int j = j0 + threadIdx.x; j <= i; j += GEN_THREADS) {
        const float e = __expf(ps[j] - mx);
        ps[j] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    __syncthreads();
    const float inv = 1.0f / sum;
    __nv_bfloat16* out = p.out + (int64_t)b * p.so.stride_b + (int64_t)i * p.so.stride_s + (int64_t)h * p.so.stride_h;
    for (int d = threadIdx.x; d < hd; d += GEN_THREADS) {
        float acc = 0.f;
        for (int j = j0; j <= i; ++j) acc += ps[j] * bf16_to_f32(row_ptr(p.v, p.sv, b, j, kvh)[d]);
        out[d] = f32_to_bf16(acc * inv);
    }
    if (threadIdx.x == 0) p.lse[((int64_t)b * p.n_heads + h) * p.seq + i] = mx + logf(sum);
}

// delta[b,h,i] = sum_d O * dO
__global__ void __launch_bounds__(GEN_THREADS) attn_generic_delta_kernel(AttnParams p, int hd) {
    dep_wait();
    const int64_t row = (int64_t)blockIdx.x * (GEN_THREADS / 32) + (threadIdx.x >> 5);
    const int64_t rows = (int64_t)p.batch * p.n_heads * p.seq;
    if (row >= rows) return;
    const int i = (int)(row % p.seq), h = (int)((row / p.seq) % p.n_heads), b = (int)(row / ((int64_t)p.seq * p.n_heads));
    const __nv_bfloat16* o = row_ptr(p.o, p.so, b, i, h);
    const __nv_bfloat16* g = row_ptr(p.d_o, p.sdo, b, i, h);
    float acc = 0.f;
    for (int d = threadIdx.x & 31; d < hd; d += 32) acc += bf16_to_f32(o[d]) * bf16_to_f32(g[d]);
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) p.delta[row] = acc;
}

// dQ[i] = scale * sum_j dS[i,j] K[j],  dS = P (dP - delta),  P = exp(scale q.k - lse),  dP = dO . V
// smem: q row [hd], dO row [hd], dS [seq]
__global__ void __launch_bounds__(GEN_THREADS) attn_generic_dq_kernel(AttnParams p, int hd) {
    dep_wait();
    extern __shared__ float sm[];
    float* qs = sm;
    float* gs = sm + hd;
    float* ds = sm + 2 * hd;
    const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, kvh = h / p.rep;
    const __nv_bfloat16* q = row_ptr(p.q, p.sq, b, i, h);
    const __nv_bfloat16* g = row_ptr(p.d_o, p.sdo, b, i, h);
    for (int d = threadIdx.x; d < hd; d += GEN_THREADS) { qs[d] = bf16_to_f32(q[d]) * p.scale; gs[d] = bf16_to_f32(g[d]); }
    __syncthreads();
    const int64_t row = ((int64_t)b * p.n_heads + h) * p.seq + i;
    const float lse = p.lse[row], delta = p.delta[row];
    const int j0 = first_visible(i, p.window);
    for (int j = j0 + threadIdx.x; j <= i; j += GEN_THREADS) {
        const __nv_bfloat16* k = row_ptr(p.k, p.sk, b, j, kvh);
        const __nv_bfloat16* v = row_ptr(p.v, p.sv, b, j, kvh);
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < hd; ++d) { s += qs[d] * bf16_to_f32(k[d]); dp += gs[d] * bf16_to_f32(v[d]); }
        ds[j] = __expf(s - lse) * (dp - delta);
    }
    __syncthreads();
    __nv_bfloat16* dq = p.dq + (int64_t)b * p.sq.stride_b + (int64_t)i * p.sq.stride_s + (int64_t)h * p.sq.stride_h;
    for (int d = threadIdx.x; d < hd; d += GEN_THREADS) {
        float acc = 0.f;
        for (int j = j0; j <= i; ++j) acc += ds[j] * bf16_to_f32(row_ptr(p.k, p.sk, b, j, kvh)[d]);
        dq[d] = f32_to_bf16(acc * p.scale);
    }
}

// dV[j] = sum_{h in group} sum_i P[i,j] dO[i],  dK[j] = scale * sum_{h in group} sum_i dS[i,j] Q[i]
// One CTA per key row; queries are processed in chunks of GEN_THREADS (one thread forms P and dS of one query, then
// the threads split the head dimension).  smem: k row [hd], v row [hd], P [GEN_THREADS], dS [GEN_THREADS]
__global__ void __launch_bounds__(GEN_THREADS) attn_generic_dkv_kernel(AttnParams p, int hd) {
    dep_wait();
    extern __shared__ float sm[];
    float* ks = sm;
    float* vs = sm + hd;
    float* pc = sm + 2 * hd;
    float* dc = pc + GEN_THREADS;
    const int j = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const __nv_bfloat16* k = row_ptr(p.k, p.sk, b, j, kvh);
    const __nv_bfloat16* v = row_ptr(p.v, p.sv, b, j, kvh);
    for (int d = threadIdx.x; d < hd; d += GEN_THREADS) { ks[d] = bf16_to_f32(k[d]); vs[d] = bf16_to_f32(v[d]); }
    __syncthreads();
    const int i_end = p.window > 0 ? min(p.seq - 1, j + p.window - 1) : p.seq - 1;       // queries i in [j, i_end] see key j
    // each thread owns the output columns d = threadIdx.x, threadIdx.x + GEN_THREADS (head sizes up to 2 * GEN_THREADS)
    float dk_acc[2] = {0.f, 0.f}, dv_acc[2] = {0.f, 0.f};
    for (int r = 0; r < p.rep; ++r) {
        const int h = kvh * p.rep + r;
        for (int i0 = j; i0 <= i_end; i0 += GEN_THREADS) {
            const int i = i0 + threadIdx.x;
            float pv = 0.f, dsv = 0.f;
            if (i <= i_end) {
                const __nv_bfloat16* q = row_ptr(p.q, p.sq, b, i, h);
                const __nv_bfloat16* g = row_ptr(p.d_o, p.sdo, b, i, h);
                float s = 0.f, dp = 0.f;
                for (int d = 0; d < hd; ++d) { s += bf16_to_f32(q[d]) * ks[d]; dp += bf16_to_f32(g[d]) * vs[d]; }
                const int64_t row = ((int64_t)b * p.n_heads + h) * p.seq + i;
                pv = __expf(s * p.scale - p.lse[row]);
                dsv = pv * (dp - p.delta[row]);
            }
            __syncthreads();
            pc[threadIdx.x] = pv;
            dc[threadIdx.x] = dsv;
            __syncthreads();
            const int n = min(GEN_THREADS, i_end - i0 + 1);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int d = threadIdx.x + c * GEN_THREADS;
                if (d >= hd) continue;
                float a = 0.f, bb = 0.f;
                for (int t = 0; t < n; ++t) {
                    a += pc[t] * bf16_to_f32(row_ptr(p.d_o, p.sdo, b, i0 + t, h)[d]);
                    bb += dc[t] * bf16_to_f32(row_ptr(p.q, p.sq, b, i0 + t, h)[d]);
                }
                dv_acc[c] += a;
                dk_acc[c] += bb;
            }
        }
    }
    __nv_bfloat16* dk = p.dk + (int64_t)b * p.sk.stride_b + (int64_t)j * p.sk.stride_s + (int64_t)kvh * p.sk.stride_h;
    __nv_bfloat16* dv = p.dv + (int64_t)b * p.sv.stride_b + (int64_t)j * p.sv.stride_s + (int64_t)kvh * p.sv.stride_h;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = threadIdx.x + c * GEN_THREADS;
        if (d < hd) { dk[d] = f32_to_bf16(dk_acc[c] * p.scale); dv[d] = f32_to_bf16(dv_acc[c]); }
    }
}

int32_t generic_limits(const AttnParams& p, int hd, size_t smem) {
    if (hd <= 0 || hd > 2 * GEN_THREADS) return fail(MFT_ERR_UNSUPPORTED, "attention: head_dim must be between 1 and 256");
    if (smem > 200 * 1024) return fail(MFT_ERR_UNSUPPORTED, "attention: sequences this long need head_dim 64, 128 or 256");
    if (p.n_heads % p.n_kv != 0) return fail(MFT_ERR_INVALID_ARG, "attention: n_heads must be a multiple of n_kv_heads");
    return MFT_OK;
}

template <typename K>
int32_t allow_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return MFT_OK;
    return check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), "attention smem attribute");
}

}  // namespace

int32_t attn_generic_fwd(const AttnParams& p, int hd, cudaStream_t stream) {
    const size_t smem = (size_t)(hd + p.seq) * 4;
    if (int32_t s = generic_limits(p, hd, smem)) return s;
    if (int32_t s = allow_smem(attn_generic_fwd_kernel, smem)) return s;
    launch_dep(attn_generic_fwd_kernel, dim3((unsigned)p.seq, (unsigned)p.n_heads, (unsigned)p.batch), dim3(GEN_THREADS), smem, stream, p, hd);
    MFT_LAUNCH_CHECK("attn_generic_fwd");
    return MFT_OK;
}

int32_t attn_generic_bwd(const AttnParams& p, int hd, cudaStream_t stream) {
    const size_t smem_dq = (size_t)(2 * hd + p.seq) * 4, smem_kv = (size_t)(2 * hd + 2 * GEN_THREADS) * 4;
    if (int32_t s = generic_limits(p, hd, smem_dq)) return s;
    if (int32_t s = allow_smem(attn_generic_dq_kernel, smem_dq)) return s;
    const int64_t rows = (int64_t)p.batch * p.n_heads * p.seq;
    launch_dep(attn_generic_delta_kernel, dim3((unsigned)((rows + GEN_THREADS / 32 - 1) / (GEN_THREADS / 32))), dim3(GEN_THREADS), (size_t)0, stream, p, hd);
    MFT_LAUNCH_CHECK("attn_generic_delta");
    launch_dep(attn_generic_dq_kernel, dim3((unsigned)p.seq, (unsigned)p.n_heads, (unsigned)p.batch), dim3(GEN_THREADS), smem_dq, stream, p, hd);
    MFT_LAUNCH_CHECK("attn_generic_dq");
    launch_dep(attn_generic_dkv_kernel, dim3((unsigned)p.seq, (unsigned)p.n_kv, (unsigned)p.batch), dim3(GEN_THREADS), smem_kv, stream, p, hd);
    MFT_LAUNCH_CHECK("attn_generic_dkv");
    return MFT_OK;
}

}  // namespace mft
