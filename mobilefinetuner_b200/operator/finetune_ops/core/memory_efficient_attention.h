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

// q, k, v: [B, heads, S, head_dim] f32 (same head count).  Composed from the fp32 operators so that
// gradients flow; the training step uses the fused flash-style kernels (mft_attn_fwd / mft_attn_bwd).
TensorPtr memory_efficient_attention(const TensorPtr& q, const TensorPtr& k, const TensorPtr& v, const TensorPtr& causal_mask = nullptr,
                                     const MemoryEfficientAttentionConfig& config = {});

}  // namespace ops
