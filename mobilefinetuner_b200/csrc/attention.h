// Parameter block shared by the attention kernels (mma.sync kernels in attention.cu, tcgen05 kernels in
// attention_sm100.cu).
#pragma once
#include "common.cuh"

namespace mft {

struct AttnParams {
    const __nv_bfloat16 *q, *k, *v, *o, *d_o;
    __nv_bfloat16 *out, *dq, *dk, *dv;
    float* lse;
    float* delta;
    float* dkv_acc;          // optional f32 [2][batch, seq, n_kv, hd] accumulator of the per-head dK/dV kernel
    mft_strides_t sq, sk, sv, so, sdo;
    int batch, seq, n_heads, n_kv, rep;
    float scale;
    int window;
};

// Forward pass on the 5th-generation tensor cores (head_dim 256, sequence a multiple of 128, token-major
// operands).  Returns MFT_ERR_UNSUPPORTED when the problem does not qualify; the caller then uses the
// mma.sync kernel.
int32_t attn_fwd_sm100(const AttnParams& p, int hd, cudaStream_t stream);
// dQ of the backward pass, same conditions.  With compute_delta the kernel also forms delta = rowsum(O * dO) and
// stores it in p.delta (for the dK/dV kernel that follows); otherwise p.delta must already hold it.
int32_t attn_dq_sm100(const AttnParams& p, int hd, bool compute_delta, cudaStream_t stream);
// dK / dV of the backward pass ADDED into p.dkv_acc (f32 [2][batch, seq, n_kv, head_dim], zeroed by the caller);
// needs p.dkv_acc and p.delta.
int32_t attn_dkv_sm100(const AttnParams& p, int hd, cudaStream_t stream);

// Any other head size (1..256): plain CUDA-core kernels, one CTA per row (attention_generic.cu).  The backward needs
// p.delta as scratch; dK / dV are written directly (p.dkv_acc is not used).
int32_t attn_generic_fwd(const AttnParams& p, int hd, cudaStream_t stream);
int32_t attn_generic_bwd(const AttnParams& p, int hd, cudaStream_t stream);

}  // namespace mft
