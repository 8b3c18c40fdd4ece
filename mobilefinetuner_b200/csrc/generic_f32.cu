// Generic fp32 kernels behind the eager `ops::` surface of the operator API:
// broadcasting element-wise arithmetic, unary maps, reductions, permutes, a
// batched fp32 matmul, row softmax, rotate-half RoPE on [B,H,S,D] tensors.
// They exist so that every public operator of the reference works on
// device-resident tensors with fp32 accuracy (its own unit tests hold 1e-5 ..
// 1e-6); the fused bf16 tensor-core kernels are what the training step uses.
#include "common.cuh"

namespace mft {
namespace {

constexpr int MAXD = 6;
struct Dims {
    int nd;
    int64_t shape[MAXD];      // output shape
    int64_t sa[MAXD];         // strides of input a (0 where broadcast)
    int64_t sb[MAXD];
};

__device__ __forceinline__ float apply_bin(int op, float a, float b) {
    switch (op) {
        case MFT_EW_ADD: return a + b;
        case MFT_EW_SUB: return a - b;
        case MFT_EW_MUL: return a * b;
        default: return a / b;
    }
}

__global__ void ew_binary_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                 int64_t n, Dims d, int same_shape) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (same_shape) { out[i] = apply_bin(op, a[i], b[i]); continue; }
        int64_t rem = i, ia = 0, ib = 0;
        for (int k = d.nd - 1; k >= 0; --k) {
            const int64_t c = rem % d.shape[k];
            rem /= d.shape[k];
            ia += c * d.sa[k];
            ib += c * d.sb[k];
        }
        out[i] = apply_bin(op, a[ia], b[ib]);
    }
}

__global__ void ew_scalar_kernel(int op, const float* __restrict__ a, float s, int scalar_first, float* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = scalar_first ? apply_bin(op, s, a[i]) : apply_bin(op, a[i], s);
}

__device__ __forceinline__ float apply_unary(int op, float x, float p) {
    switch (op) {
        case MFT_UN_GELU: return gelu_tanh_f(x);
        case MFT_UN_GELU_GRAD: return gelu_tanh_grad_f(x);
        case MFT_UN_SILU: return x / (1.0f + expf(-x));
        case MFT_UN_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case MFT_UN_TANH: return tanhf(x);
        case MFT_UN_RELU: return x > 0.f ? x : 0.f;
        case MFT_UN_EXP: return expf(x);
        case MFT_UN_LOG: return logf(x);
        case MFT_UN_SQRT: return sqrtf(x);
        case MFT_UN_ABS: return fabsf(x);
        case MFT_UN_POW: return powf(x, p);
        case MFT_UN_NEG: return -x;
        default: return x;
    }
}
__global__ void ew_unary_kernel(int op, const float* __restrict__ a, float p, float* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = apply_unary(op, a[i], p);
}

// out[o, i] = sum_r in[o, r, i]
__global__ void reduce_sum_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t outer, int64_t red, int64_t inner, float scale) {
    const int64_t total = outer * inner;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t o = idx / inner, i = idx % inner;
        const float* p = in + o * red * inner + i;
        float acc = 0.f;
        for (int64_t r = 0; r < red; ++r) acc += p[r * inner];
        out[idx] = acc * scale;
    }
}

struct Perm {
    int nd;
    int64_t out_shape[MAXD];
    int64_t in_stride[MAXD];   // stride in the input of the dimension that became output dim k
};
__global__ void permute_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int64_t n, Perm p) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, src = 0;
        for (int k = p.nd - 1; k >= 0; --k) {
            src += (rem % p.out_shape[k]) * p.in_stride[k];
            rem /= p.out_shape[k];
        }
        out[i] = in[src];
    }
}

// C[b] (M x N) = A[b] (M x K) * op(B[b]) ; B is [K,N] (trans_b = 0) or [N,K] (trans_b = 1); fp32 FMA, 32x32 tiles.
__global__ void matmul_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                                  int64_t stride_a, int64_t stride_b, int64_t stride_c, int trans_b) {
    __shared__ float As[32][33], Bs[32][33];
    const int b = blockIdx.z;
    const float* a = A + b * stride_a;
    const float* bb = B + b * stride_b;
    float* c = C + b * stride_c;
    const int row = blockIdx.y * 32 + threadIdx.y, col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        As[threadIdx.y][threadIdx.x] = (row < M && ka < K) ? a[(int64_t)row * K + ka] : 0.f;
        float bv = 0.f;
        if (kb < K && col < N) bv = trans_b ? bb[(int64_t)col * K + kb] : bb[(int64_t)kb * N + col];
        Bs[threadIdx.y][threadIdx.x] = bv;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; ++k) acc = fmaf(As[threadIdx.y][k], Bs[k][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < M && col < N) c[(int64_t)row * N + col] = acc;
}

__global__ void softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t dim) {
    __shared__ float scratch[32];
    __shared__ float bmax;
    const float* xr = x + (int64_t)blockIdx.x * dim;
    float* yr = y + (int64_t)blockIdx.x * dim;
    float m = -INFINITY;
    for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) m = fmaxf(m, xr[i]);
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
    for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) s += expf(xr[i] - m);
    s = block_sum(s, scratch);
    const float inv = 1.0f / s;
    for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) yr[i] = expf(xr[i] - m) * inv;
}
// dx = y * (dy - sum(dy * y))
__global__ void softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ dy, float* __restrict__ dx, int64_t dim) {
    __shared__ float scratch[32];
    const int64_t off = (int64_t)blockIdx.x * dim;
    float dot = 0.f;
    for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) dot += y[off + i] * dy[off + i];
    dot = block_sum(dot, scratch);
    for (int64_t i = threadIdx.x; i < dim; i += blockDim.x) dx[off + i] = y[off + i] * (dy[off + i] - dot);
}

// rotate-half RoPE on [rows = B*H, S, D]; sign = +1 forward, -1 backward (transposed rotation)
__global__ void rope_f32_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ cs, const float* __restrict__ sn,
                                int64_t S, int64_t D, int64_t total_pairs, float sign) {
    const int64_t half = D / 2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_pairs; i += stride) {
        const int64_t d = i % half, pos = (i / half) % S, row = i / (half * S);
        const int64_t base = (row * S + pos) * D;
        const float c = cs[pos * half + d], s = sn[pos * half + d] * sign;
        const float x1 = x[base + d], x2 = x[base + half + d];
        y[base + d] = x1 * c - x2 * s;
        y[base + half + d] = x1 * s + x2 * c;
    }
}

__global__ void swiglu_f32_kernel(const float* __restrict__ g, const float* __restrict__ u, const float* __restrict__ dy,
                                  float* __restrict__ o1, float* __restrict__ o2, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float s = 1.0f / (1.0f + expf(-g[i]));
        if (!dy) { o1[i] = g[i] * s * u[i]; continue; }
        o1[i] = dy[i] * u[i] * (s * (1.0f + g[i] * (1.0f - s)));
        o2[i] = dy[i] * g[i] * s;
    }
}

inline int grid1(int64_t n) { int64_t b = (n + 255) / 256; return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b)); }

}  // namespace
}  // namespace mft

using namespace mft;

extern "C" {

int32_t mft_ew_binary_f32(int32_t op, const float* a, const int64_t* a_shape, int32_t a_nd, const float* b, const int64_t* b_shape,
                          int32_t b_nd, float* out, const int64_t* out_shape, int32_t out_nd, mft_stream_t stream) {
    MFT_CHECK_ARG(a && b && out && out_nd >= 0 && out_nd <= MAXD && a_nd <= out_nd && b_nd <= out_nd, "mft_ew_binary_f32: bad argument");
    MFT_CHECK_ARG(op >= MFT_EW_ADD && op <= MFT_EW_DIV, "mft_ew_binary_f32: unknown op");
    Dims d{};
    d.nd = out_nd;
    int64_t n = 1;
    bool same = (a_nd == out_nd && b_nd == out_nd);
    for (int k = 0; k < out_nd; ++k) { d.shape[k] = out_shape[k]; n *= out_shape[k]; }
    // right-aligned broadcasting, contiguous inputs
    int64_t sa = 1, sb = 1;
    for (int k = out_nd - 1; k >= 0; --k) {
        const int ka = k - (out_nd - a_nd), kb = k - (out_nd - b_nd);
        const int64_t da = ka >= 0 ? a_shape[ka] : 1, db = kb >= 0 ? b_shape[kb] : 1;
        MFT_CHECK_ARG((da == out_shape[k] || da == 1) && (db == out_shape[k] || db == 1), "mft_ew_binary_f32: shapes do not broadcast");
        d.sa[k] = da == 1 ? 0 : sa;
        d.sb[k] = db == 1 ? 0 : sb;
        if (da != out_shape[k] || db != out_shape[k]) same = false;
        sa *= da; sb *= db;
    }
    if (n == 0) return MFT_OK;
    ew_binary_kernel<<<grid1(n), 256, 0, as_stream(stream)>>>(op, a, b, out, n, d, same ? 1 : 0);
    MFT_LAUNCH_CHECK("ew_binary_f32");
    return MFT_OK;
}

int32_t mft_ew_scalar_f32(int32_t op, const float* a, float scalar, int32_t scalar_first, float* out, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(a && out && n >= 0 && op >= MFT_EW_ADD && op <= MFT_EW_DIV, "mft_ew_scalar_f32: bad argument");
    if (n == 0) return MFT_OK;
    ew_scalar_kernel<<<grid1(n), 256, 0, as_stream(stream)>>>(op, a, scalar, scalar_first, out, n);
    MFT_LAUNCH_CHECK("ew_scalar_f32");
    return MFT_OK;
}

int32_t mft_ew_unary_f32(int32_t op, const float* a, float param, float* out, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(a && out && n >= 0 && op >= MFT_UN_GELU && op <= MFT_UN_COPY, "mft_ew_unary_f32: bad argument");
    if (n == 0) return MFT_OK;
    ew_unary_kernel<<<grid1(n), 256, 0, as_stream(stream)>>>(op, a, param, out, n);
    MFT_LAUNCH_CHECK("ew_unary_f32");
    return MFT_OK;
}

int32_t mft_reduce_sum_f32(const float* in, float* out, int64_t outer, int64_t reduce, int64_t inner, float scale, mft_stream_t stream) {
    MFT_CHECK_ARG(in && out && outer > 0 && reduce > 0 && inner > 0, "mft_reduce_sum_f32: bad argument");
    reduce_sum_kernel<<<grid1(outer * inner), 256, 0, as_stream(stream)>>>(in, out, outer, reduce, inner, scale);
    MFT_LAUNCH_CHECK("reduce_sum_f32");
    return MFT_OK;
}

int32_t mft_permute_b32(const void* in, void* out, const int64_t* in_shape, const int32_t* perm, int32_t nd, mft_stream_t stream) {
    MFT_CHECK_ARG(in && out && in_shape && perm && nd >= 1 && nd <= MAXD, "mft_permute_b32: bad argument");
    int64_t in_stride[MAXD];
    int64_t s = 1;
    for (int k = nd - 1; k >= 0; --k) { in_stride[k] = s; s *= in_shape[k]; }
    Perm p{};
    p.nd = nd;
    int64_t n = 1;
    for (int k = 0; k < nd; ++k) {
        MFT_CHECK_ARG(perm[k] >= 0 && perm[k] < nd, "mft_permute_b32: bad permutation");
        p.out_shape[k] = in_shape[perm[k]];
        p.in_stride[k] = in_stride[perm[k]];
        n *= p.out_shape[k];
    }
    if (n == 0) return MFT_OK;
    permute_kernel<<<grid1(n), 256, 0, as_stream(stream)>>>((const uint32_t*)in, (uint32_t*)out, n, p);
    MFT_LAUNCH_CHECK("permute_b32");
    return MFT_OK;
}

int32_t mft_matmul_f32(const float* a, const float* b, float* c, int64_t batch, int64_t m, int64_t n, int64_t k, int64_t stride_a,
                       int64_t stride_b, int64_t stride_c, int32_t trans_b, mft_stream_t stream) {
    MFT_CHECK_ARG(a && b && c && batch > 0 && m > 0 && n > 0 && k > 0 && batch <= 65535, "mft_matmul_f32: bad argument");
    dim3 grid((unsigned)((n + 31) / 32), (unsigned)((m + 31) / 32), (unsigned)batch);
    MFT_CHECK_ARG(grid.y <= 65535, "mft_matmul_f32: M too large");
    matmul_f32_kernel<<<grid, dim3(32, 32), 0, as_stream(stream)>>>(a, b, c, (int)m, (int)n, (int)k, stride_a, stride_b, stride_c, trans_b);
    MFT_LAUNCH_CHECK("matmul_f32");
    return MFT_OK;
}

int32_t mft_softmax_f32(const float* x, float* y, int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(x && y && rows > 0 && dim > 0, "mft_softmax_f32: bad argument");
    softmax_fwd_kernel<<<(unsigned)rows, 128, 0, as_stream(stream)>>>(x, y, dim);
    MFT_LAUNCH_CHECK("softmax_f32");
    return MFT_OK;
}
int32_t mft_softmax_bwd_f32(const float* y, const float* dy, float* dx, int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(y && dy && dx && rows > 0 && dim > 0, "mft_softmax_bwd_f32: bad argument");
    softmax_bwd_kernel<<<(unsigned)rows, 128, 0, as_stream(stream)>>>(y, dy, dx, dim);
    MFT_LAUNCH_CHECK("softmax_bwd_f32");
    return MFT_OK;
}

int32_t mft_rope_f32(const float* x, float* y, const float* cos_tab, const float* sin_tab, int64_t rows, int64_t seq, int64_t head_dim,
                     int32_t backward, mft_stream_t stream) {
    MFT_CHECK_ARG(x && y && cos_tab && sin_tab && rows > 0 && seq > 0 && head_dim > 0 && head_dim % 2 == 0, "mft_rope_f32: bad argument");
    const int64_t pairs = rows * seq * (head_dim / 2);
    rope_f32_kernel<<<grid1(pairs), 256, 0, as_stream(stream)>>>(x, y, cos_tab, sin_tab, seq, head_dim, pairs, backward ? -1.0f : 1.0f);
    MFT_LAUNCH_CHECK("rope_f32");
    return MFT_OK;
}

int32_t mft_swiglu_f32(const float* gate, const float* up, const float* dy, float* out1, float* out2, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(gate && up && out1 && n > 0 && (!dy || out2), "mft_swiglu_f32: bad argument");
    swiglu_f32_kernel<<<grid1(n), 256, 0, as_stream(stream)>>>(gate, up, dy, out1, out2, n);
    MFT_LAUNCH_CHECK("swiglu_f32");
    return MFT_OK;
}

}  // extern "C"
