// RMSNorm / LayerNorm forward and backward, and the fused per-head
// RMSNorm + rotary embedding used on Q and K.  Model-width RMSNorm rows up to
// 2048 elements are handled one WARP per row (all of the row's 128-bit loads
// in flight at once, shuffle reductions, no block barrier); wider rows and
// LayerNorm use one CTA per row.  The row stays in registers between the
// reduction and the write.  One warp per (token, head) for the per-head
// kernel.  HBM-bound: every element is read once and written once.
#include <cmath>
#include <vector>

#include "common.cuh"

namespace mft {

constexpr int NORM_THREADS = 128;
constexpr int NORM_VPT = 4;   // up to 4 x 8 elements cached per thread -> dim <= 4096 with 128 threads

template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr int v = MFT_F32; };
template <> struct dtype_of<__nv_bfloat16> { static constexpr int v = MFT_BF16; };

// ---------------------------------------------------------------- RMSNorm forward
template <typename TX, typename TY>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, float eps, int unit_offset,
                   TY* __restrict__ y, float* __restrict__ rstd_out, const float* __restrict__ residual,
                   float* __restrict__ sum_out, int64_t dim) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const TX* xr = x + row * dim;
    const int nvec = (int)(dim / 8);
    float v[NORM_VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            load8(xr + i * 8, v[k]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)dim + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float wv[8], o[8];
            load8(w + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rstd * (unit_offset ? 1.0f + wv[j] : wv[j]);
            if (y) store8(y + row * dim + i * 8, o);
            if (residual) {
                float r[8];
                load8(residual + row * dim + i * 8, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] += o[j];
                store8(sum_out + row * dim + i * 8, r);
            }
        }
    }
}

// ---------------------------------------------------------------- RMSNorm backward
// g = dy * w_eff ; dx = g*rstd - x * rstd^3/D * sum(g*x)
template <typename TDY, typename TX, typename TDX>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ rstd_in, float eps, int unit_offset, TDX* __restrict__ dx,
                   int accumulate, float* __restrict__ dweight, int64_t dim) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int nvec = (int)(dim / 8);
    float xv[NORM_VPT][8], g[NORM_VPT][8];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float wv[8];
            load8(x + row * dim + i * 8, xv[k]);
            load8(dy + row * dim + i * 8, g[k]);
            load8(w + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (dweight) atomicAdd(dweight + i * 8 + j, g[k][j] * xv[k][j] * (rstd_in ? rstd_in[row] : 0.f));
                g[k][j] *= (unit_offset ? 1.0f + wv[j] : wv[j]);
                dot += g[k][j] * xv[k][j];
                ss += xv[k][j] * xv[k][j];
            }
        }
    }
    dot = block_sum(dot, scratch);
    float rstd;
    if (rstd_in) rstd = rstd_in[row];
    else {
        ss = block_sum(ss, scratch);
        rstd = rsqrtf(ss / (float)dim + eps);
    }
    const float coeff = rstd * rstd * rstd / (float)dim * dot;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = g[k][j] * rstd - xv[k][j] * coeff;
            if (accumulate) {
                float prev[8];
                load8(dx + row * dim + i * 8, prev);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += prev[j];
            }
            store8(dx + row * dim + i * 8, o);
        }
    }
}


// ---------------------------------------------------------------- RMSNorm, one warp per row (dim <= 256 * VPL)
constexpr int NORM_WARPS = 8;     // rows per CTA

template <typename TX, typename TY, int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_fwd_warp_kernel(const TX* __restrict__ x, const float* __restrict__ w, float eps, int unit_offset,
                        TY* __restrict__ y, float* __restrict__ rstd_out, const float* __restrict__ residual,
                        float* __restrict__ sum_out, int64_t rows, int64_t dim) {
    dep_trigger();
    dep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const TX* xr = x + row * dim;
    const int nvec = (int)(dim / 8);
    float v[VPL][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) load8(xr + i * 8, v[k]);
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        if (lane + k * 32 < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
        }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)dim + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8], o[8];
            load8(w + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rstd * (unit_offset ? 1.0f + wv[j] : wv[j]);
            if (y) store8(y + row * dim + i * 8, o);
            if (residual) {
                float r[8];
                load8(residual + row * dim + i * 8, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] += o[j];
                store8(sum_out + row * dim + i * 8, r);
            }
        }
    }
}

template <typename TDY, typename TX, typename TDX, int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_bwd_warp_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ rstd_in, float eps, int unit_offset, TDX* __restrict__ dx,
                        int accumulate, float* __restrict__ dweight, int64_t rows, int64_t dim) {
    dep_trigger();
    dep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nvec = (int)(dim / 8);
    float xv[VPL][8], g[VPL][8];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            load8(x + row * dim + i * 8, xv[k]);
            load8(dy + row * dim + i * 8, g[k]);
        }
    }
    const float rs_in = rstd_in ? rstd_in[row] : 0.f;
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8];
            load8(w + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (dweight) atomicAdd(dweight + i * 8 + j, g[k][j] * xv[k][j] * rs_in);
                g[k][j] *= (unit_offset ? 1.0f + wv[j] : wv[j]);
                dot += g[k][j] * xv[k][j];
                ss += xv[k][j] * xv[k][j];
            }
        }
    }
    dot = warp_sum(dot);
    float rstd = rs_in;
    if (!rstd_in) rstd = rsqrtf(warp_sum(ss) / (float)dim + eps);
    const float coeff = rstd * rstd * rstd / (float)dim * dot;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = g[k][j] * rstd - xv[k][j] * coeff;
            if (accumulate) {
                float prev[8];
                load8(dx + row * dim + i * 8, prev);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += prev[j];
            }
            store8(dx + row * dim + i * 8, o);
        }
    }
}


// Ask for the 32 bytes at p early (no register is held): the fused norm kernels read some rows only after a
// warp reduction, and without this their latency adds to that of the first loads.
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" :: "l"(p)); }

// ---------------------------------------------------------------- fused post-norm + residual add + next pre-norm
// Gemma wraps every block as  x_sum = x + rms(y_branch) ,  h_next = rms(x_sum)  (post-norm of one block, residual
// add, pre-norm of the next).  One warp per row keeps x_sum in registers between the two norms, so x_sum is
// written once and never re-read: same arithmetic, in the same order, as the two separate kernels.
template <int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_add_norm_fwd_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w_post, int unit_post,
                            const float* __restrict__ residual, const float* __restrict__ w_next, int unit_next, float eps,
                            float* __restrict__ sum_out, float* __restrict__ rstd_post, __nv_bfloat16* __restrict__ h_next,
                            float* __restrict__ rstd_next, int64_t rows, int64_t dim) {
    dep_trigger();
    dep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nvec = (int)(dim / 8);
    float v[VPL][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) load8(y + row * dim + i * 8, v[k]);
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) prefetch_l1(residual + row * dim + i * 8);
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k)
        if (lane + k * 32 < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
        }
    ss = warp_sum(ss);
    const float rp = rsqrtf(ss / (float)dim + eps);
    if (lane == 0) rstd_post[row] = rp;
    float ss2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8], r[8];
            load8(w_post + i * 8, wv);
            load8(residual + row * dim + i * 8, r);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float o = v[k][j] * rp * (unit_post ? 1.0f + wv[j] : wv[j]);
                v[k][j] = r[j] + o;
            }
            store8(sum_out + row * dim + i * 8, v[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k)
        if (lane + k * 32 < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ss2 += v[k][j] * v[k][j];
        }
    ss2 = warp_sum(ss2);
    const float rn = rsqrtf(ss2 / (float)dim + eps);
    if (lane == 0) rstd_next[row] = rn;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8], o[8];
            load8(w_next + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[k][j] * rn * (unit_next ? 1.0f + wv[j] : wv[j]);
            store8(h_next + row * dim + i * 8, o);
        }
    }
}

// Backward of the same pair: dx (f32, the gradient on x_sum that came down the residual path) first receives the
// gradient through the next pre-norm (dy_next), is stored, and then goes through the post-norm of the branch.
template <int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_pair_bwd_kernel(const __nv_bfloat16* __restrict__ dy_next, const float* __restrict__ x_sum, const float* __restrict__ w_next,
                        int unit_next, const float* __restrict__ rstd_next, float* __restrict__ dx,
                        const __nv_bfloat16* __restrict__ y_branch, const float* __restrict__ w_post, int unit_post,
                        const float* __restrict__ rstd_post, __nv_bfloat16* __restrict__ d_branch, int64_t rows, int64_t dim) {
    dep_trigger();
    dep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nvec = (int)(dim / 8);
    float xv[VPL][8], g[VPL][8];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            load8(x_sum + row * dim + i * 8, xv[k]);
            load8(dy_next + row * dim + i * 8, g[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            prefetch_l1(dx + row * dim + i * 8);
            if ((i & 1) == 0) prefetch_l1(y_branch + row * dim + i * 8);      // 16-byte pieces: every other lane names a new 32 bytes
        }
    }
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8];
            load8(w_next + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                g[k][j] *= (unit_next ? 1.0f + wv[j] : wv[j]);
                dot += g[k][j] * xv[k][j];
            }
        }
    }
    dot = warp_sum(dot);
    const float rn = rstd_next[row];
    const float coeff = rn * rn * rn / (float)dim * dot;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float prev[8];
            load8(dx + row * dim + i * 8, prev);
#pragma unroll
            for (int j = 0; j < 8; ++j) g[k][j] = (g[k][j] * rn - xv[k][j] * coeff) + prev[j];
            store8(dx + row * dim + i * 8, g[k]);
        }
    }
    // post-norm of the branch: dy = the dx row just formed
    float dot2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float wv[8];
            load8(y_branch + row * dim + i * 8, xv[k]);
            load8(w_post + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                g[k][j] *= (unit_post ? 1.0f + wv[j] : wv[j]);
                dot2 += g[k][j] * xv[k][j];
            }
        }
    }
    dot2 = warp_sum(dot2);
    const float rp = rstd_post[row];
    const float coeff2 = rp * rp * rp / (float)dim * dot2;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = g[k][j] * rp - xv[k][j] * coeff2;
            store8(d_branch + row * dim + i * 8, o);
        }
    }
}

// ---------------------------------------------------------------- LayerNorm
template <typename TX, typename TY>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                     TY* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t dim) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int nvec = (int)(dim / 8);
    float v[NORM_VPT][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            load8(x + row * dim + i * 8, v[k]);
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[k][j];
        }
    }
    const float mean = block_sum(s, scratch) / (float)dim;
    float var = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { float d = v[k][j] - mean; var += d * d; }
        }
    }
    var = block_sum(var, scratch) / (float)dim;
    const float rstd = 1.0f / sqrtf(var + eps);
    if (threadIdx.x == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float wv[8], bv[8], o[8];
            load8(w + i * 8, wv);
            load8(b + i * 8, bv);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd * wv[j] + bv[j];
            store8(y + row * dim + i * 8, o);
        }
    }
}

// dx = rstd/D * (D*g - sum(g) - xhat*sum(g*xhat)),  g = dy*w
template <typename TDY, typename TX, typename TDX>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in, TDX* __restrict__ dx,
                     int accumulate, float* __restrict__ dweight, float* __restrict__ dbias, int64_t dim) {
    dep_trigger();
    dep_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int nvec = (int)(dim / 8);
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NORM_VPT][8], g[NORM_VPT][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float wv[8];
            load8(x + row * dim + i * 8, xh[k]);
            load8(dy + row * dim + i * 8, g[k]);
            load8(w + i * 8, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xh[k][j] = (xh[k][j] - mean) * rstd;
                if (dweight) atomicAdd(dweight + i * 8 + j, g[k][j] * xh[k][j]);
                if (dbias) atomicAdd(dbias + i * 8 + j, g[k][j]);
                g[k][j] *= wv[j];
                sg += g[k][j];
                sgx += g[k][j] * xh[k][j];
            }
        }
    }
    sg = block_sum(sg, scratch);
    sgx = block_sum(sgx, scratch);
    const float D = (float)dim;
#pragma unroll
    for (int k = 0; k < NORM_VPT; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < nvec) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (rstd / D) * (D * g[k][j] - sg - xh[k][j] * sgx);
            if (accumulate) {
                float prev[8];
                load8(dx + row * dim + i * 8, prev);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += prev[j];
            }
            store8(dx + row * dim + i * 8, o);
        }
    }
}

// ---------------------------------------------------------------- per-head norm + RoPE
// PER consecutive elements in one access when VEC (the launcher has checked the alignment), one by one otherwise.
template <int PER, bool VEC>
__device__ __forceinline__ void ld_bf16_run(const __nv_bfloat16* p, float (&v)[PER]) {
    if constexpr (VEC && PER == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
    } else if constexpr (VEC && PER == 2) {
        const __nv_bfloat162 u = *reinterpret_cast<const __nv_bfloat162*>(p);
        v[0] = __low2float(u); v[1] = __high2float(u);
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) v[j] = bf16_to_f32(p[j]);
    }
}
template <int PER, bool VEC>
__device__ __forceinline__ void st_bf16_run(__nv_bfloat16* p, const float (&v)[PER]) {
    if constexpr (VEC && PER == 4) {
        const __nv_bfloat162 lo = __halves2bfloat162(f32_to_bf16(v[0]), f32_to_bf16(v[1])), hi = __halves2bfloat162(f32_to_bf16(v[2]), f32_to_bf16(v[3]));
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&lo); u.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    } else if constexpr (VEC && PER == 2) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __halves2bfloat162(f32_to_bf16(v[0]), f32_to_bf16(v[1]));
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) p[j] = f32_to_bf16(v[j]);
    }
}
template <int PER, bool VEC>
__device__ __forceinline__ void ld_f32_run(const float* p, float (&v)[PER]) {
    if constexpr (VEC && PER == 4) {
        const float4 u = __ldg(reinterpret_cast<const float4*>(p));
        v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
    } else if constexpr (VEC && PER == 2) {
        const float2 u = __ldg(reinterpret_cast<const float2*>(p));
        v[0] = u.x; v[1] = u.y;
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) v[j] = __ldg(p + j);
    }
}

// One warp per (token, head).  Lane l owns PER = head_dim/64 consecutive
// elements of the first half (d = l*PER ..) and the paired elements d + hd/2.
template <int PER, bool BWD, bool VEC>
__global__ void headnorm_rope_kernel(const __nv_bfloat16* __restrict__ in, int64_t ld_in,   // fwd: x ; bwd: dy
                                     const __nv_bfloat16* __restrict__ x, int64_t ld_x,     // bwd only: forward input
                                     const float* __restrict__ nw, float eps,
                                     float* __restrict__ rstd_buf,                           // fwd: out ; bwd: in
                                     const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                     __nv_bfloat16* __restrict__ out, int64_t ld_out,
                                     int64_t n_tokens, int64_t seq_len, int64_t n_heads) {
    dep_trigger();
    dep_wait();
    constexpr int HD = PER * 64, HALF = PER * 32;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= n_tokens * n_heads) return;
    const int64_t tok = wid / n_heads, head = wid % n_heads;
    const int64_t pos = tok % seq_len;
    const int d0 = lane * PER;
    float a[PER], b[PER];   // first-half / second-half values of `in`
    {
        const __nv_bfloat16* p = in + tok * ld_in + head * HD;
        ld_bf16_run<PER, VEC>(p + d0, a);
        ld_bf16_run<PER, VEC>(p + HALF + d0, b);
    }
    float c[PER], s[PER];
    if (cos_tab) {
        ld_f32_run<PER, VEC>(cos_tab + pos * HALF + d0, c);
        ld_f32_run<PER, VEC>(sin_tab + pos * HALF + d0, s);
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) { c[j] = 1.f; s[j] = 0.f; }
    }
    float w1[PER], w2[PER];
    if (nw) {
        ld_f32_run<PER, VEC>(nw + d0, w1);
        ld_f32_run<PER, VEC>(nw + HALF + d0, w2);
#pragma unroll
        for (int j = 0; j < PER; ++j) { w1[j] = 1.0f + w1[j]; w2[j] = 1.0f + w2[j]; }
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) { w1[j] = 1.0f; w2[j] = 1.0f; }
    }
    __nv_bfloat16* o = out + tok * ld_out + head * HD;
    if (!BWD) {
        float rstd = 1.0f;
        if (nw) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < PER; ++j) ss += a[j] * a[j] + b[j] * b[j];
            ss = warp_sum(ss);
            rstd = rsqrtf(ss / (float)HD + eps);
            if (lane == 0 && rstd_buf) rstd_buf[wid] = rstd;
        }
        float y1[PER], y2[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const float x1 = a[j] * rstd * w1[j], x2 = b[j] * rstd * w2[j];
            y1[j] = x1 * c[j] - x2 * s[j];
            y2[j] = x1 * s[j] + x2 * c[j];
        }
        st_bf16_run<PER, VEC>(o + d0, y1);
        st_bf16_run<PER, VEC>(o + HALF + d0, y2);
    } else {
        // undo the rotation: dxn1 = dy1*c + dy2*s ; dxn2 = -dy1*s + dy2*c
        float g1[PER], g2[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            g1[j] = a[j] * c[j] + b[j] * s[j];
            g2[j] = -a[j] * s[j] + b[j] * c[j];
        }
        if (nw) {
            const __nv_bfloat16* xp = x + tok * ld_x + head * HD;
            float x1[PER], x2[PER];
            float dot = 0.f;
            ld_bf16_run<PER, VEC>(xp + d0, x1);
            ld_bf16_run<PER, VEC>(xp + HALF + d0, x2);
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                g1[j] *= w1[j]; g2[j] *= w2[j];
                dot += g1[j] * x1[j] + g2[j] * x2[j];
            }
            dot = warp_sum(dot);
            const float rstd = rstd_buf[wid];
            const float coeff = rstd * rstd * rstd / (float)HD * dot;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                g1[j] = g1[j] * rstd - x1[j] * coeff;
                g2[j] = g2[j] * rstd - x2[j] * coeff;
            }
        }
        st_bf16_run<PER, VEC>(o + d0, g1);
        st_bf16_run<PER, VEC>(o + HALF + d0, g2);
    }
}

// Same operation for any even head size (test-sized models: 4, 8, 16, ... wide heads): one warp per (token, head),
// lanes stride over the pairs (d, d + hd/2), scalar accesses only.
template <bool BWD>
__global__ void headnorm_rope_any_kernel(const __nv_bfloat16* __restrict__ in, int64_t ld_in, const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                         const float* __restrict__ nw, float eps, float* __restrict__ rstd_buf,
                                         const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                         __nv_bfloat16* __restrict__ out, int64_t ld_out, int64_t n_tokens, int64_t seq_len, int64_t n_heads, int hd) {
    dep_trigger();
    dep_wait();
    const int half = hd / 2;
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= n_tokens * n_heads) return;
    const int64_t tok = wid / n_heads, head = wid % n_heads, pos = tok % seq_len;
    const __nv_bfloat16* p = in + tok * ld_in + head * hd;
    __nv_bfloat16* o = out + tok * ld_out + head * hd;
    if (!BWD) {
        float rstd = 1.0f;
        if (nw) {
            float ss = 0.f;
            for (int d = lane; d < hd; d += 32) { const float v = bf16_to_f32(p[d]); ss += v * v; }
            ss = warp_sum(ss);
            rstd = rsqrtf(ss / (float)hd + eps);
            if (lane == 0 && rstd_buf) rstd_buf[wid] = rstd;
        }
        for (int d = lane; d < half; d += 32) {
            const float c = cos_tab ? cos_tab[pos * half + d] : 1.f, sn = sin_tab ? sin_tab[pos * half + d] : 0.f;
            const float x1 = bf16_to_f32(p[d]) * rstd * (nw ? 1.0f + nw[d] : 1.0f);
            const float x2 = bf16_to_f32(p[half + d]) * rstd * (nw ? 1.0f + nw[half + d] : 1.0f);
            o[d] = f32_to_bf16(x1 * c - x2 * sn);
            o[half + d] = f32_to_bf16(x1 * sn + x2 * c);
        }
    } else {
        const __nv_bfloat16* xp = nw ? x + tok * ld_x + head * hd : nullptr;
        float dot = 0.f;
        if (nw)
            for (int d = lane; d < half; d += 32) {
                const float c = cos_tab ? cos_tab[pos * half + d] : 1.f, sn = sin_tab ? sin_tab[pos * half + d] : 0.f;
                const float a = bf16_to_f32(p[d]), b = bf16_to_f32(p[half + d]);
                const float g1 = (a * c + b * sn) * (1.0f + nw[d]), g2 = (-a * sn + b * c) * (1.0f + nw[half + d]);
                dot += g1 * bf16_to_f32(xp[d]) + g2 * bf16_to_f32(xp[half + d]);
            }
        dot = warp_sum(dot);
        const float rstd = nw ? rstd_buf[wid] : 1.0f;
        const float coeff = nw ? rstd * rstd * rstd / (float)hd * dot : 0.f;
        for (int d = lane; d < half; d += 32) {
            const float c = cos_tab ? cos_tab[pos * half + d] : 1.f, sn = sin_tab ? sin_tab[pos * half + d] : 0.f;
            const float a = bf16_to_f32(p[d]), b = bf16_to_f32(p[half + d]);
            float g1 = a * c + b * sn, g2 = -a * sn + b * c;
            if (nw) {
                g1 = g1 * (1.0f + nw[d]) * rstd - bf16_to_f32(xp[d]) * coeff;
                g2 = g2 * (1.0f + nw[half + d]) * rstd - bf16_to_f32(xp[half + d]) * coeff;
            }
            o[d] = f32_to_bf16(g1);
            o[half + d] = f32_to_bf16(g2);
        }
    }
}

}  // namespace mft

using namespace mft;

#define DISPATCH_2(XD, YD, CALL)                                                         \
    if (XD == MFT_F32 && YD == MFT_F32) { CALL(float, float) }                           \
    else if (XD == MFT_F32 && YD == MFT_BF16) { CALL(float, __nv_bfloat16) }             \
    else if (XD == MFT_BF16 && YD == MFT_F32) { CALL(__nv_bfloat16, float) }             \
    else if (XD == MFT_BF16 && YD == MFT_BF16) { CALL(__nv_bfloat16, __nv_bfloat16) }    \
    else return fail(MFT_ERR_INVALID_ARG, "dtype must be MFT_F32 or MFT_BF16");

extern "C" {

int32_t mft_rmsnorm_fwd(const void* x, int32_t xd, const float* w, float eps, int32_t unit_offset, void* y, int32_t yd,
                        float* rstd, const float* residual, float* sum_out, int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(x && w && rows > 0 && dim > 0, "mft_rmsnorm_fwd: bad argument");
    MFT_CHECK_ARG(y || (residual && sum_out), "mft_rmsnorm_fwd: nothing to write");
    MFT_CHECK_ARG(!residual || sum_out, "mft_rmsnorm_fwd: residual needs sum_out");
    MFT_CHECK_ARG(dim % 8 == 0 && dim <= 8 * NORM_THREADS * NORM_VPT, "mft_rmsnorm_fwd: dim must be a multiple of 8 and <= 4096");
    const unsigned wblocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
#define WCALL(TX, TY, VPL) launch_dep(rmsnorm_fwd_warp_kernel<TX, TY, VPL>, dim3(wblocks), dim3(NORM_WARPS * 32), (size_t)(0), as_stream(stream), (const TX*)x, w, eps, unit_offset, (TY*)y, rstd, residual, sum_out, rows, dim);
#define CALL(TX, TY)                                                                                     \
    if (dim <= 1280) { WCALL(TX, TY, 5) }                                                                \
    else if (dim <= 2048) { WCALL(TX, TY, 8) }                                                           \
    else launch_dep(rmsnorm_fwd_kernel<TX, TY>, dim3((unsigned)rows), dim3(NORM_THREADS), (size_t)(0), as_stream(stream), (const TX*)x, w, eps, unit_offset, (TY*)y, rstd, residual, sum_out, dim);
    DISPATCH_2(xd, yd, CALL)
#undef CALL
#undef WCALL
    MFT_LAUNCH_CHECK("rmsnorm_fwd");
    return MFT_OK;
}

int32_t mft_rmsnorm_bwd(const void* dy, int32_t dyd, const void* x, int32_t xd, const float* w, const float* rstd, float eps,
                        int32_t unit_offset, void* dx, int32_t dxd, int32_t accumulate, float* dweight, int64_t rows,
                        int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(dy && x && w && dx && rows > 0 && dim > 0, "mft_rmsnorm_bwd: bad argument");
    MFT_CHECK_ARG(dim % 8 == 0 && dim <= 8 * NORM_THREADS * NORM_VPT, "mft_rmsnorm_bwd: dim must be a multiple of 8 and <= 4096");
    MFT_CHECK_ARG(!accumulate || dxd == MFT_F32, "mft_rmsnorm_bwd: accumulate needs f32 dx");
    MFT_CHECK_ARG(!dweight || rstd, "mft_rmsnorm_bwd: dweight needs rstd");
    const unsigned wblocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
#define WLAUNCH(TDY, TX, TDX, VPL) launch_dep(rmsnorm_bwd_warp_kernel<TDY, TX, TDX, VPL>, dim3(wblocks), dim3(NORM_WARPS * 32), (size_t)(0), as_stream(stream), (const TDY*)dy, (const TX*)x, w, rstd, eps, unit_offset, (TDX*)dx, accumulate, dweight, rows, dim);
#define LAUNCH(TDY, TX, TDX)                                                                             \
    if (dim <= 1280) { WLAUNCH(TDY, TX, TDX, 5) }                                                        \
    else if (dim <= 2048) { WLAUNCH(TDY, TX, TDX, 8) }                                                   \
    else launch_dep(rmsnorm_bwd_kernel<TDY, TX, TDX>, dim3((unsigned)rows), dim3(NORM_THREADS), (size_t)(0), as_stream(stream), (const TDY*)dy, (const TX*)x, w, rstd, eps, unit_offset, (TDX*)dx, accumulate, dweight, dim);
#define CALL(TDY, TX) if (dxd == MFT_F32) { LAUNCH(TDY, TX, float) } else if (dxd == MFT_BF16) { LAUNCH(TDY, TX, __nv_bfloat16) } else return fail(MFT_ERR_INVALID_ARG, "mft_rmsnorm_bwd: bad dx dtype");
    DISPATCH_2(dyd, xd, CALL)
#undef CALL
#undef LAUNCH
#undef WLAUNCH
    MFT_LAUNCH_CHECK("rmsnorm_bwd");
    return MFT_OK;
}

int32_t mft_rmsnorm_add_norm_fwd(const void* y_bf16, const float* w_post, int32_t unit_post, const float* residual,
                                 const float* w_next, int32_t unit_next, float eps, float* sum_out, float* rstd_post,
                                 void* h_next_bf16, float* rstd_next, int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(y_bf16 && w_post && residual && w_next && sum_out && rstd_post && h_next_bf16 && rstd_next && rows > 0, "mft_rmsnorm_add_norm_fwd: bad argument");
    MFT_CHECK_ARG(dim > 0 && dim % 8 == 0, "mft_rmsnorm_add_norm_fwd: dim must be a multiple of 8");
    if (dim > 2048) return fail(MFT_ERR_UNSUPPORTED, "mft_rmsnorm_add_norm_fwd: rows wider than 2048 use the separate norm calls");
    const unsigned wblocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
#define FCALL(VPL) launch_dep(rmsnorm_add_norm_fwd_kernel<VPL>, dim3(wblocks), dim3(NORM_WARPS * 32), (size_t)0, as_stream(stream), \
                              (const __nv_bfloat16*)y_bf16, w_post, (int)unit_post, residual, w_next, (int)unit_next, eps, sum_out, rstd_post, \
                              (__nv_bfloat16*)h_next_bf16, rstd_next, rows, dim)
    if (dim <= 1280) FCALL(5); else FCALL(8);
#undef FCALL
    MFT_LAUNCH_CHECK("rmsnorm_add_norm_fwd");
    return MFT_OK;
}

int32_t mft_rmsnorm_pair_bwd(const void* dy_next_bf16, const float* x_sum, const float* w_next, int32_t unit_next,
                             const float* rstd_next, float* dx_inout, const void* y_branch_bf16, const float* w_post,
                             int32_t unit_post, const float* rstd_post, void* d_branch_bf16, int64_t rows, int64_t dim,
                             mft_stream_t stream) {
    MFT_CHECK_ARG(dy_next_bf16 && x_sum && w_next && rstd_next && dx_inout && y_branch_bf16 && w_post && rstd_post && d_branch_bf16 && rows > 0,
                  "mft_rmsnorm_pair_bwd: bad argument");
    MFT_CHECK_ARG(dim > 0 && dim % 8 == 0, "mft_rmsnorm_pair_bwd: dim must be a multiple of 8");
    if (dim > 2048) return fail(MFT_ERR_UNSUPPORTED, "mft_rmsnorm_pair_bwd: rows wider than 2048 use the separate norm calls");
    const unsigned wblocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
#define BCALL(VPL) launch_dep(rmsnorm_pair_bwd_kernel<VPL>, dim3(wblocks), dim3(NORM_WARPS * 32), (size_t)0, as_stream(stream), \
                              (const __nv_bfloat16*)dy_next_bf16, x_sum, w_next, (int)unit_next, rstd_next, dx_inout, \
                              (const __nv_bfloat16*)y_branch_bf16, w_post, (int)unit_post, rstd_post, (__nv_bfloat16*)d_branch_bf16, rows, dim)
    if (dim <= 1280) BCALL(5); else BCALL(8);
#undef BCALL
    MFT_LAUNCH_CHECK("rmsnorm_pair_bwd");
    return MFT_OK;
}

int32_t mft_layernorm_fwd(const void* x, int32_t xd, const float* w, const float* b, float eps, void* y, int32_t yd,
                          float* mean, float* rstd, int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(x && w && b && y && rows > 0 && dim > 0, "mft_layernorm_fwd: bad argument");
    MFT_CHECK_ARG(dim % 8 == 0 && dim <= 8 * NORM_THREADS * NORM_VPT, "mft_layernorm_fwd: dim must be a multiple of 8 and <= 4096");
#define CALL(TX, TY) launch_dep(layernorm_fwd_kernel<TX, TY>, dim3((unsigned)rows), dim3(NORM_THREADS), (size_t)(0), as_stream(stream), (const TX*)x, w, b, eps, (TY*)y, mean, rstd, dim);
    DISPATCH_2(xd, yd, CALL)
#undef CALL
    MFT_LAUNCH_CHECK("layernorm_fwd");
    return MFT_OK;
}

int32_t mft_layernorm_bwd(const void* dy, int32_t dyd, const void* x, int32_t xd, const float* w, const float* mean,
                          const float* rstd, void* dx, int32_t dxd, int32_t accumulate, float* dweight, float* dbias,
                          int64_t rows, int64_t dim, mft_stream_t stream) {
    MFT_CHECK_ARG(dy && x && w && mean && rstd && dx && rows > 0 && dim > 0, "mft_layernorm_bwd: bad argument");
    MFT_CHECK_ARG(dim % 8 == 0 && dim <= 8 * NORM_THREADS * NORM_VPT, "mft_layernorm_bwd: dim must be a multiple of 8 and <= 4096");
    MFT_CHECK_ARG(!accumulate || dxd == MFT_F32, "mft_layernorm_bwd: accumulate needs f32 dx");
#define LAUNCH(TDY, TX, TDX) launch_dep(layernorm_bwd_kernel<TDY, TX, TDX>, dim3((unsigned)rows), dim3(NORM_THREADS), (size_t)(0), as_stream(stream), (const TDY*)dy, (const TX*)x, w, mean, rstd, (TDX*)dx, accumulate, dweight, dbias, dim);
#define CALL(TDY, TX) if (dxd == MFT_F32) { LAUNCH(TDY, TX, float) } else if (dxd == MFT_BF16) { LAUNCH(TDY, TX, __nv_bfloat16) } else return fail(MFT_ERR_INVALID_ARG, "mft_layernorm_bwd: bad dx dtype");
    DISPATCH_2(dyd, xd, CALL)
#undef CALL
#undef LAUNCH
    MFT_LAUNCH_CHECK("layernorm_bwd");
    return MFT_OK;
}

int32_t mft_rope_table_host(float* cos_host, float* sin_host, int64_t seq_len, int64_t head_dim, float theta) {
    MFT_CHECK_ARG(cos_host && sin_host && seq_len > 0 && head_dim > 0 && head_dim % 2 == 0, "mft_rope_table_host: bad argument");
    const int64_t half = head_dim / 2;
    for (int64_t pos = 0; pos < seq_len; ++pos)
        for (int64_t d = 0; d < half; ++d) {
            // identical expression (and float types) to apply_rope in the reference
            float freq = 1.0f / std::pow(theta, 2.0f * d / head_dim);
            float angle = pos * freq;
            cos_host[pos * half + d] = std::cos(angle);
            sin_host[pos * half + d] = std::sin(angle);
        }
    return MFT_OK;
}

static int32_t launch_headnorm_rope(bool bwd, const void* in, int64_t ld_in, const void* x, int64_t ld_x, const float* nw,
                                    float eps, float* rstd, const float* cos_tab, const float* sin_tab, void* out,
                                    int64_t ld_out, int64_t n_tokens, int64_t seq_len, int64_t n_heads, int64_t hd,
                                    mft_stream_t stream) {
    const int64_t warps = n_tokens * n_heads;
    const int threads = 256;
    const unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
    // one 4- / 8-byte access per run of a lane's elements when every operand allows it
    auto al = [](const void* p, uintptr_t a) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % a == 0; };
    const bool vec = al(in, 8) && al(x, 8) && al(out, 8) && al(nw, 16) && al(cos_tab, 16) && al(sin_tab, 16) && ld_in % 4 == 0 &&
                     ld_out % 4 == 0 && (x == nullptr || ld_x % 4 == 0);
#define HL(PER, B) do { if (vec) HL2(PER, B, true); else HL2(PER, B, false); } while (0)
#define HL2(PER, B, V) launch_dep(headnorm_rope_kernel<PER, B, V>, dim3(blocks), dim3(threads), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)in, ld_in, (const __nv_bfloat16*)x, ld_x, nw, eps, rstd, cos_tab, sin_tab, (__nv_bfloat16*)out, ld_out, n_tokens, seq_len, n_heads)
    if (hd == 64) { if (bwd) HL2(1, true, false); else HL2(1, false, false); }
    else if (hd == 128) { if (bwd) HL(2, true); else HL(2, false); }
    else if (hd == 256) { if (bwd) HL(4, true); else HL(4, false); }
    else if (hd > 0 && hd % 2 == 0 && hd <= 4096) {
        if (bwd) launch_dep(headnorm_rope_any_kernel<true>, dim3(blocks), dim3(threads), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)in, ld_in, (const __nv_bfloat16*)x, ld_x, nw, eps, rstd, cos_tab, sin_tab, (__nv_bfloat16*)out, ld_out, n_tokens, seq_len, n_heads, (int)hd);
        else launch_dep(headnorm_rope_any_kernel<false>, dim3(blocks), dim3(threads), (size_t)(0), as_stream(stream), (const __nv_bfloat16*)in, ld_in, (const __nv_bfloat16*)x, ld_x, nw, eps, rstd, cos_tab, sin_tab, (__nv_bfloat16*)out, ld_out, n_tokens, seq_len, n_heads, (int)hd);
    }
    else return fail(MFT_ERR_UNSUPPORTED, "headnorm_rope: head_dim must be even");
#undef HL
#undef HL2
    MFT_LAUNCH_CHECK("headnorm_rope");
    return MFT_OK;
}

int32_t mft_headnorm_rope_fwd(const void* x, int64_t ld, const float* nw, float eps, const float* cos_tab,
                              const float* sin_tab, void* y, int64_t ld_y, float* rstd, int64_t n_tokens, int64_t seq_len,
                              int64_t n_heads, int64_t hd, mft_stream_t stream) {
    MFT_CHECK_ARG(x && y && n_tokens > 0 && seq_len > 0 && n_heads > 0, "mft_headnorm_rope_fwd: bad argument");
    MFT_CHECK_ARG((cos_tab == nullptr) == (sin_tab == nullptr), "mft_headnorm_rope_fwd: cos and sin tables go together");
    MFT_CHECK_ARG(!nw || rstd, "mft_headnorm_rope_fwd: norm needs an rstd buffer");
    return launch_headnorm_rope(false, x, ld, nullptr, 0, nw, eps, rstd, cos_tab, sin_tab, y, ld_y, n_tokens, seq_len, n_heads, hd, stream);
}
int32_t mft_headnorm_rope_bwd(const void* dy, int64_t ld_dy, const void* x, int64_t ld, const float* nw, const float* rstd,
                              const float* cos_tab, const float* sin_tab, void* dx, int64_t ld_dx, int64_t n_tokens,
                              int64_t seq_len, int64_t n_heads, int64_t hd, mft_stream_t stream) {
    MFT_CHECK_ARG(dy && dx && n_tokens > 0 && seq_len > 0 && n_heads > 0, "mft_headnorm_rope_bwd: bad argument");
    MFT_CHECK_ARG(!nw || (rstd && x), "mft_headnorm_rope_bwd: norm needs x and rstd");
    return launch_headnorm_rope(true, dy, ld_dy, x, ld, nw, 0.f, const_cast<float*>(rstd), cos_tab, sin_tab, dx, ld_dx, n_tokens, seq_len, n_heads, hd, stream);
}

}  // extern "C"
