// Attention entry point of the reference's core/memory_efficient_attention.h.
#pragma once
#include "tensor.h"

namespace ops {

struct MemoryEfficientAttentionConfig {
    bool use_causal_mask = true;
    float scale = -1.0f;          // < 0: 1/sqrt(head_dim)
    int chunk_size = 512;
    bool save_probs = false;
};

// q, k, v: [B, heads, S, head_dim] f32.  With the bf16 compute type (ops::set_compute_dtype) and a causal mask this
// is the fused flash-style kernel pair mft_attn_fwd / mft_attn_bwd (k / v may then hold fewer heads than q: grouped
// queries); with the fp32 compute type it is composed from the fp32 operators (same head count), to fp32 accuracy.
TensorPtr memory_efficient_attention(const TensorPtr& q, const TensorPtr& k, const TensorPtr& v, const TensorPtr& causal_mask = nullptr,
                                     const MemoryEfficientAttentionConfig& config = {});

}  // namespace ops
