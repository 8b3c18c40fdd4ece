// Memory-bound kernels of the LoRA step: casts / transposes, embedding gather,
// activations (GELU, SwiGLU, GeGLU) forward and backward, residual adds,
// repeat_kv, the table-driven LoRA panel pack/unpack and the Adam update.
// All of them are HBM-bound: 128-bit accesses, grid-stride loops, no reuse.
#include "act_math.cuh"
#include "common.cuh"

#include <atomic>

namespace mft {

static inline int grid_for(int64_t work_items, int threads, int max_blocks = 148 * 16) {
    int64_t b = (work_items + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > max_blocks) b = max_blocks;
    return (int)b;
}

// ---------------------------------------------------------------- casts
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
    dep_trigger();
    dep_wait();
    const int64_t nv = n / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float v[8];
        load8(src + i * 8, v);
        store8(dst + i * 8, v);
    }
    for (int64_t i = nv * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = f32_to_bf16(src[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n) {
    dep_trigger();
    dep_wait();
    const int64_t nv = n / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float v[8];
        load8(src + i * 8, v);
        store8(dst + i * 8, v);
    }
    for (int64_t i = nv * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = bf16_to_f32(src[i]);
}

// dst[c, r] = (bf16) src[r, c]; 32x32 tiles through padded shared memory.
template <typename TS>
__global__ void transpose_to_bf16_kernel(const TS* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                         int64_t rows, int64_t cols, int64_t dst_ld) {
    dep_trigger();
    dep_wait();
    __shared__ float tile[32][33];
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int64_t r = r0 + j, c = c0 + threadIdx.x;
        float v = 0.f;
        if (r < rows && c < cols) {
            if constexpr (sizeof(TS) == 4) v = src[r * cols + c];
            else v = bf16_to_f32(src[r * cols + c]);
        }
        tile[j][threadIdx.x] = v;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int64_t c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[c * dst_ld + r] = f32_to_bf16(tile[threadIdx.x][j]);
    }
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 const __nv_bfloat16* __restrict__ pos, float* __restrict__ out,
                                 int64_t seq_len, int64_t hidden, int64_t vocab, float scale,
                                 int32_t* __restrict__ status) {
    dep_trigger();
    dep_wait();
    const int64_t t = blockIdx.x;
    const int32_t id = ids[t];
    float* o = out + t * hidden;
    if (id < 0 || id >= vocab) {
        if (status && threadIdx.x == 0) atomicExch(status, MFT_ERR_BOUNDS);
        for (int64_t i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const __nv_bfloat16* row = table + (int64_t)id * hidden;
    const __nv_bfloat16* prow = pos ? pos + (t % seq_len) * hidden : nullptr;
    const int64_t nv = hidden / 8;
    for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
        float v[8];
        load8(row + i * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= scale;
        if (prow) {
            float p[8];
            load8(prow + i * 8, p);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += p[j];
        }
        store8(o + i * 8, v);
    }
    for (int64_t i = nv * 8 + threadIdx.x; i < hidden; i += blockDim.x) {
        float v = bf16_to_f32(row[i]) * scale;
        if (prow) v += bf16_to_f32(prow[i]);
        o[i] = v;
    }
}

// ---------------------------------------------------------------- activations
template <int KIND>
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                               int64_t ld, __nv_bfloat16* __restrict__ y, int64_t rows, int64_t cols) {
    dep_trigger();
    dep_wait();
    const int64_t vpr = cols / 8;
    const int64_t total = rows * vpr;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / vpr, c = (i % vpr) * 8;
        float g[8], u[8], o[8];
        load8(gate + r * ld + c, g);
        if (KIND != MFT_ACT_GELU) load8(up + r * ld + c, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (KIND == MFT_ACT_GELU) o[j] = gelu_tanh_fast(g[j]);
            else o[j] = glu_fwd(KIND == MFT_ACT_GEGLU, g[j], u[j]);
        }
        store8(y + r * cols + c, o);
    }
}
template <int KIND>
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gate,
                               const __nv_bfloat16* __restrict__ up, int64_t ld,
                               __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                               int64_t rows, int64_t cols) {
    dep_trigger();
    dep_wait();
    const int64_t vpr = cols / 8;
    const int64_t total = rows * vpr;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / vpr, c = (i % vpr) * 8;
        float g[8], u[8], d[8], dg[8], du[8];
        load8(gate + r * ld + c, g);
        load8(dy + r * cols + c, d);
        if (KIND != MFT_ACT_GELU) load8(up + r * ld + c, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (KIND == MFT_ACT_GELU) {
                float val, grad;
                gelu_tanh_both(g[j], val, grad);
                dg[j] = d[j] * grad;
            } else {
                glu_bwd(KIND == MFT_ACT_GEGLU, d[j], g[j], u[j], dg[j], du[j]);     // the same code as the GEMM epilogue that fuses it
            }
        }
        store8(dgate + r * ld + c, dg);
        if (KIND != MFT_ACT_GELU) store8(dup + r * ld + c, du);
    }
}

template <typename TB>
__global__ void add_kernel(const float* __restrict__ a, const TB* __restrict__ b, float* __restrict__ out, int64_t n) {
    dep_trigger();
    dep_wait();
    const int64_t nv = n / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float x[8], y[8];
        load8(a + i * 8, x);
        load8(b + i * 8, y);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += y[j];
        store8(out + i * 8, x);
    }
    for (int64_t i = nv * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float bv;
        if constexpr (sizeof(TB) == 4) bv = b[i]; else bv = bf16_to_f32(b[i]);
        out[i] = a[i] + bv;
    }
}
__global__ void scale_kernel(float* __restrict__ x, float alpha, int64_t n) {
    dep_trigger();
    dep_wait();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] *= alpha;
}

// ---------------------------------------------------------------- repeat_kv
template <typename T>
__global__ void repeat_kv_kernel(const T* __restrict__ kv, T* __restrict__ out, int64_t n_kv, int64_t seq,
                                 int64_t hd, int64_t rep, int64_t total) {
    dep_trigger();
    dep_wait();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t d = i % hd, s = (i / hd) % seq, h = (i / (hd * seq)) % (n_kv * rep), b = i / (hd * seq * n_kv * rep);
        out[i] = kv[((b * n_kv + h / rep) * seq + s) * hd + d];
    }
}
__global__ void repeat_kv_bwd_kernel(const float* __restrict__ dout, float* __restrict__ dkv, int64_t n_kv,
                                     int64_t seq, int64_t hd, int64_t rep, int64_t total) {
    dep_trigger();
    dep_wait();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t d = i % hd, s = (i / hd) % seq, h = (i / (hd * seq)) % n_kv, b = i / (hd * seq * n_kv);
        float acc = 0.f;
        for (int64_t r = 0; r < rep; ++r) acc += dout[((b * n_kv * rep + h * rep + r) * seq + s) * hd + d];
        dkv[i] = acc;
    }
}

// ---------------------------------------------------------------- LoRA panel pack / unpack
template <bool ACCUM_F32>
__global__ void block_copy_kernel(const mft_block_copy_t* __restrict__ table) {
    dep_trigger();
    dep_wait();
    const mft_block_copy_t e = table[blockIdx.x];
    const int64_t total = (int64_t)e.rows * e.cols;
    const float* src = static_cast<const float*>(e.src);
    for (int64_t i = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.y * blockDim.x) {
        const int64_t r = i / e.cols, c = i % e.cols;
        const float v = src[r * e.src_ld + c];
        const int64_t di = e.transpose ? c * (int64_t)e.dst_ld + r : r * (int64_t)e.dst_ld + c;
        if (ACCUM_F32) static_cast<float*>(e.dst)[di] += v;
        else static_cast<__nv_bfloat16*>(e.dst)[di] = f32_to_bf16(v);
    }
}

// ---------------------------------------------------------------- optimizer
// Sum of squares with a result that does not depend on the order in which blocks finish (data-parallel replicas
// clip by this norm and must stay bit-identical): every block leaves its partial sum in a slot of a static array,
// the block that arrives last adds the partials in index order and adds the total to *out.  Calls that may overlap on
// the device use different slots (the host hands them out round-robin).
constexpr int SQ_SLOTS = 16, SQ_MAX_BLOCKS = 1024;
__device__ float sq_partials[SQ_SLOTS][SQ_MAX_BLOCKS];
__device__ unsigned int sq_arrived[SQ_SLOTS];
__global__ void sqnorm_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ out, int slot) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    __shared__ int last;
    float acc = 0.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc += g[i] * g[i];
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) {
        sq_partials[slot][blockIdx.x] = acc;
        __threadfence();
        last = atomicAdd(&sq_arrived[slot], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    float total = 0.f;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) total += *reinterpret_cast<volatile float*>(&sq_partials[slot][i]);
    __syncthreads();                          // scratch is reused
    total = block_sum(total, scratch);
    if (threadIdx.x == 0) {
        *out += total;
        sq_arrived[slot] = 0;                 // ready for the next call that gets this slot
    }
}
static int next_sq_slot() {
    static std::atomic<unsigned> counter{0};
    return (int)(counter.fetch_add(1) % SQ_SLOTS);
}
__global__ void adam_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                            int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                            const float* __restrict__ sqnorm, float max_norm, float clip_eps, int zero_grad) {
    dep_trigger();
    dep_wait();
    float clip = 1.0f;
    if (sqnorm != nullptr && max_norm > 0.f) {
        const float norm = sqrtf(*sqnorm);
        if (norm > max_norm) clip = max_norm / (norm + clip_eps);
    }
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gv = g[i] * clip;
        const float pv = p[i];
        if (wd > 0.f) gv += wd * pv;
        const float mv = b1 * m[i] + (1.0f - b1) * gv;
        const float vv = b2 * v[i] + (1.0f - b2) * gv * gv;
        m[i] = mv;
        v[i] = vv;
        p[i] = pv - lr * (mv / bc1) / (sqrtf(vv / bc2) + eps);
        if (zero_grad) g[i] = 0.f;
    }
}

}  // namespace mft

using namespace mft;

extern "C" {

int32_t mft_cast_f32_to_bf16(const float* src, void* dst, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(src && dst && n >= 0, "mft_cast_f32_to_bf16: bad argument");
    if (n == 0) return MFT_OK;
    launch_dep(cast_f32_bf16_kernel, dim3(grid_for(n / 8 + 1, 256)), dim3(256), (size_t)(0), as_stream(stream), src, (__nv_bfloat16*)dst, n);
    MFT_LAUNCH_CHECK("cast_f32_bf16");
    return MFT_OK;
}
int32_t mft_cast_bf16_to_f32(const void* src, float* dst, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(src && dst && n >= 0, "mft_cast_bf16_to_f32: bad argument");
    if (n == 0) return MFT_OK;
    launch_dep(cast_bf16_f32_kernel, dim3(grid_for(n / 8 + 1, 256)), dim3(256), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)src, dst, n);
    MFT_LAUNCH_CHECK("cast_bf16_f32");
    return MFT_OK;
}
int32_t mft_transpose_f32_to_bf16(const float* src, void* dst, int64_t rows, int64_t cols, mft_stream_t stream) {
    MFT_CHECK_ARG(src && dst && rows > 0 && cols > 0, "mft_transpose_f32_to_bf16: bad argument");
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    MFT_CHECK_ARG(grid.y <= 65535, "mft_transpose_f32_to_bf16: too many rows");
    launch_dep(transpose_to_bf16_kernel<float>, dim3(grid), dim3(dim3(32, 8)), (size_t)(0), as_stream(stream), src, (__nv_bfloat16*)dst, rows, cols, rows);
    MFT_LAUNCH_CHECK("transpose_f32_bf16");
    return MFT_OK;
}
int32_t mft_transpose_bf16(const void* src, void* dst, int64_t rows, int64_t cols, mft_stream_t stream) {
    return mft_transpose_bf16_ld(src, dst, rows, cols, rows, stream);
}
int32_t mft_transpose_bf16_ld(const void* src, void* dst, int64_t rows, int64_t cols, int64_t dst_ld, mft_stream_t stream) {
    MFT_CHECK_ARG(src && dst && rows > 0 && cols > 0 && dst_ld >= rows, "mft_transpose_bf16_ld: bad argument");
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    MFT_CHECK_ARG(grid.y <= 65535, "mft_transpose_bf16_ld: too many rows");
    launch_dep(transpose_to_bf16_kernel<__nv_bfloat16>, dim3(grid), dim3(dim3(32, 8)), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, rows, cols, dst_ld);
    MFT_LAUNCH_CHECK("transpose_bf16");
    return MFT_OK;
}

int32_t mft_embedding_gather(const int32_t* ids, const void* table, const void* pos, float* out, int64_t n_tokens,
                             int64_t seq_len, int64_t hidden, int64_t vocab, float scale, int32_t* status_dev,
                             mft_stream_t stream) {
    MFT_CHECK_ARG(ids && table && out && n_tokens > 0 && hidden > 0 && vocab > 0 && seq_len > 0, "mft_embedding_gather: bad argument");
    MFT_CHECK_ARG(hidden % 8 == 0, "mft_embedding_gather: hidden must be a multiple of 8");
    launch_dep(embedding_kernel, dim3((unsigned)n_tokens), dim3(128), (size_t)(0), as_stream(stream), ids, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos, out,
                                                                        seq_len, hidden, vocab, scale, status_dev);
    MFT_LAUNCH_CHECK("embedding_gather");
    return MFT_OK;
}

int32_t mft_act_fwd(int32_t kind, const void* gate, const void* up, int64_t ld, void* y, int64_t rows, int64_t cols,
                    mft_stream_t stream) {
    MFT_CHECK_ARG(gate && y && rows > 0 && cols > 0 && cols % 8 == 0 && ld % 8 == 0, "mft_act_fwd: bad argument (cols and ld must be multiples of 8)");
    MFT_CHECK_ARG(kind == MFT_ACT_GELU || up, "mft_act_fwd: gated activation needs `up`");
    const int g = grid_for(rows * cols / 8, 256);
    auto G = (const __nv_bfloat16*)gate; auto U = (const __nv_bfloat16*)up; auto Y = (__nv_bfloat16*)y;
    if (kind == MFT_ACT_GELU) launch_dep(act_fwd_kernel<MFT_ACT_GELU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), G, U, ld, Y, rows, cols);
    else if (kind == MFT_ACT_SWIGLU) launch_dep(act_fwd_kernel<MFT_ACT_SWIGLU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), G, U, ld, Y, rows, cols);
    else if (kind == MFT_ACT_GEGLU) launch_dep(act_fwd_kernel<MFT_ACT_GEGLU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), G, U, ld, Y, rows, cols);
    else return fail(MFT_ERR_INVALID_ARG, "mft_act_fwd: unknown kind");
    MFT_LAUNCH_CHECK("act_fwd");
    return MFT_OK;
}
int32_t mft_act_bwd(int32_t kind, const void* dy, const void* gate, const void* up, int64_t ld, void* dgate, void* dup,
                    int64_t rows, int64_t cols, mft_stream_t stream) {
    MFT_CHECK_ARG(dy && gate && dgate && rows > 0 && cols > 0 && cols % 8 == 0 && ld % 8 == 0, "mft_act_bwd: bad argument");
    MFT_CHECK_ARG(kind == MFT_ACT_GELU || (up && dup), "mft_act_bwd: gated activation needs `up` and `dup`");
    const int g = grid_for(rows * cols / 8, 256);
    auto D = (const __nv_bfloat16*)dy; auto G = (const __nv_bfloat16*)gate; auto U = (const __nv_bfloat16*)up;
    auto DG = (__nv_bfloat16*)dgate; auto DU = (__nv_bfloat16*)dup;
    if (kind == MFT_ACT_GELU) launch_dep(act_bwd_kernel<MFT_ACT_GELU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), D, G, U, ld, DG, DU, rows, cols);
    else if (kind == MFT_ACT_SWIGLU) launch_dep(act_bwd_kernel<MFT_ACT_SWIGLU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), D, G, U, ld, DG, DU, rows, cols);
    else if (kind == MFT_ACT_GEGLU) launch_dep(act_bwd_kernel<MFT_ACT_GEGLU>, dim3(g), dim3(256), (size_t)(0), as_stream(stream), D, G, U, ld, DG, DU, rows, cols);
    else return fail(MFT_ERR_INVALID_ARG, "mft_act_bwd: unknown kind");
    MFT_LAUNCH_CHECK("act_bwd");
    return MFT_OK;
}
int32_t mft_add_f32(const float* a, const float* b, float* out, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(a && b && out && n > 0, "mft_add_f32: bad argument");
    launch_dep(add_kernel<float>, dim3(grid_for(n / 8 + 1, 256)), dim3(256), (size_t)(0), as_stream(stream), a, b, out, n);
    MFT_LAUNCH_CHECK("add_f32");
    return MFT_OK;
}
int32_t mft_add_f32_bf16(const float* a, const void* b, float* out, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(a && b && out && n > 0, "mft_add_f32_bf16: bad argument");
    launch_dep(add_kernel<__nv_bfloat16>, dim3(grid_for(n / 8 + 1, 256)), dim3(256), (size_t)(0), as_stream(stream), a, (const __nv_bfloat16*)b, out, n);
    MFT_LAUNCH_CHECK("add_f32_bf16");
    return MFT_OK;
}
int32_t mft_scale_f32(float* x, float alpha, int64_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(x && n > 0, "mft_scale_f32: bad argument");
    launch_dep(scale_kernel, dim3(grid_for(n, 256)), dim3(256), (size_t)(0), as_stream(stream), x, alpha, n);
    MFT_LAUNCH_CHECK("scale_f32");
    return MFT_OK;
}

int32_t mft_repeat_kv(const void* kv, int32_t dtype, void* out, int64_t batch, int64_t n_kv, int64_t seq, int64_t hd,
                      int64_t rep, mft_stream_t stream) {
    MFT_CHECK_ARG(kv && out && batch > 0 && n_kv > 0 && seq > 0 && hd > 0 && rep > 0, "mft_repeat_kv: bad argument");
    const int64_t total = batch * n_kv * rep * seq * hd;
    if (dtype == MFT_F32) launch_dep(repeat_kv_kernel<float>, dim3(grid_for(total, 256)), dim3(256), (size_t)(0), as_stream(stream), (const float*)kv, (float*)out, n_kv, seq, hd, rep, total);
    else if (dtype == MFT_BF16) launch_dep(repeat_kv_kernel<__nv_bfloat16>, dim3(grid_for(total, 256)), dim3(256), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)kv, (__nv_bfloat16*)out, n_kv, seq, hd, rep, total);
    else return fail(MFT_ERR_INVALID_ARG, "mft_repeat_kv: dtype must be f32 or bf16");
    MFT_LAUNCH_CHECK("repeat_kv");
    return MFT_OK;
}
int32_t mft_repeat_kv_bwd(const float* dout, float* dkv, int64_t batch, int64_t n_kv, int64_t seq, int64_t hd, int64_t rep,
                          mft_stream_t stream) {
    MFT_CHECK_ARG(dout && dkv && batch > 0 && n_kv > 0 && seq > 0 && hd > 0 && rep > 0, "mft_repeat_kv_bwd: bad argument");
    const int64_t total = batch * n_kv * seq * hd;
    launch_dep(repeat_kv_bwd_kernel, dim3(grid_for(total, 256)), dim3(256), (size_t)(0), as_stream(stream), dout, dkv, n_kv, seq, hd, rep, total);
    MFT_LAUNCH_CHECK("repeat_kv_bwd");
    return MFT_OK;
}

int32_t mft_pack_blocks_bf16(const mft_block_copy_t* table_dev, int32_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(table_dev && n >= 0, "mft_pack_blocks_bf16: bad argument");
    if (n == 0) return MFT_OK;
    launch_dep(block_copy_kernel<false>, dim3(dim3((unsigned)n, 8)), dim3(256), (size_t)(0), as_stream(stream), table_dev);
    MFT_LAUNCH_CHECK("pack_blocks_bf16");
    return MFT_OK;
}
int32_t mft_accumulate_blocks_f32(const mft_block_copy_t* table_dev, int32_t n, mft_stream_t stream) {
    MFT_CHECK_ARG(table_dev && n >= 0, "mft_accumulate_blocks_f32: bad argument");
    if (n == 0) return MFT_OK;
    launch_dep(block_copy_kernel<true>, dim3(dim3((unsigned)n, 8)), dim3(256), (size_t)(0), as_stream(stream), table_dev);
    MFT_LAUNCH_CHECK("accumulate_blocks_f32");
    return MFT_OK;
}

int32_t mft_grad_sqnorm(const float* grads, int64_t n, float* sqnorm_dev, mft_stream_t stream) {
    MFT_CHECK_ARG(grads && sqnorm_dev && n > 0, "mft_grad_sqnorm: bad argument");
    if (int32_t s = check_cuda(cudaMemsetAsync(sqnorm_dev, 0, 4, as_stream(stream)), "sqnorm memset")) return s;
    launch_dep(sqnorm_kernel, dim3(grid_for(n, 256, 148 * 4)), dim3(256), (size_t)(0), as_stream(stream), grads, n, sqnorm_dev, next_sq_slot());
    MFT_LAUNCH_CHECK("grad_sqnorm");
    return MFT_OK;
}
int32_t mft_grad_sqnorm_add(const float* grads, int64_t n, float* sqnorm_dev, mft_stream_t stream) {
    MFT_CHECK_ARG(grads && sqnorm_dev && n > 0, "mft_grad_sqnorm_add: bad argument");
    launch_dep(sqnorm_kernel, dim3(grid_for(n, 256, 148 * 4)), dim3(256), (size_t)(0), as_stream(stream), grads, n, sqnorm_dev, next_sq_slot());
    MFT_LAUNCH_CHECK("grad_sqnorm_add");
    return MFT_OK;
}
int32_t mft_adam_step(float* params, float* grads, float* m, float* v, int64_t n, int64_t step, float lr, float beta1,
                      float beta2, float eps, float wd, const float* sqnorm_dev, float max_norm, float clip_eps,
                      int32_t zero_grad, mft_stream_t stream) {
    MFT_CHECK_ARG(params && grads && m && v && n > 0 && step >= 1, "mft_adam_step: bad argument");
    // bias corrections exactly as the reference computes them: 1 - powf(beta, step)
    const float bc1 = 1.0f - powf(beta1, (float)step);
    const float bc2 = 1.0f - powf(beta2, (float)step);
    launch_dep(adam_kernel, dim3(grid_for(n, 256)), dim3(256), (size_t)(0), as_stream(stream), params, grads, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                                  sqnorm_dev, max_norm, clip_eps, zero_grad);
    MFT_LAUNCH_CHECK("adam_step");
    return MFT_OK;
}

}  // extern "C"
