// Element-wise math of the gated activations, shared by the stand-alone activation kernels and the GEMM epilogues
// that fuse them (gelu: core/ops.cpp:1243-1267 / GeluBackward backward_functions.cpp:164-186, tanh form;
// swiglu: ops.cpp:2416-2452 / SwiGLUBackward :277-295).
#pragma once
#include "common.cuh"

namespace mft {

// bf16 in / bf16 out: the hardware tanh approximation (relative error ~2^-11) is below the output rounding
// (2^-9), and keeps these kernels at memory speed; the f32 operators use the exact tanhf.
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// value and derivative of the tanh-form GELU from one tanh
__device__ __forceinline__ void gelu_tanh_both(float x, float& val, float& grad) {
    const float x2 = x * x;
    const float t = tanh_fast(0.7978845608f * (x + 0.044715f * x * x2));
    const float dt = 0.7978845608f * (1.0f + 3.0f * 0.044715f * x2);
    val = 0.5f * x * (1.0f + t);
    grad = 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * dt;
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    return 0.5f * x * (1.0f + tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x)));
}
// logistic function from the hardware exponential and reciprocal (two special-function instructions; an IEEE
// division costs ~10 more instructions per element, which shows in the GEMM epilogues that fuse the gating).
// Relative error ~2^-21, far below the bf16 rounding of the result; exp overflow gives 1 / inf = 0, the right limit.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
// act = f(gate) * up with f = gelu (geglu != 0) or silu
__device__ __forceinline__ float glu_fwd(bool geglu, float g, float u) {
    return geglu ? gelu_tanh_fast(g) * u : g * sigmoid_fast(g) * u;
}
__device__ __forceinline__ void glu_bwd(bool geglu, float d, float g, float u, float& dg, float& du) {
    if (geglu) {
        float val, grad;
        gelu_tanh_both(g, val, grad);
        dg = d * u * grad;
        du = d * val;
    } else {
        const float s = sigmoid_fast(g);
        dg = d * u * (s * (1.0f + g * (1.0f - s)));
        du = d * g * s;
    }
}

}  // namespace mft
