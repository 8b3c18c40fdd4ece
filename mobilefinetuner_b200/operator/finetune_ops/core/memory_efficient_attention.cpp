#include "memory_efficient_attention.h"

#include <cmath>

#include "ops.h"

namespace ops {

TensorPtr memory_efficient_attention(const TensorPtr& q, const TensorPtr& k, const TensorPtr& v, const TensorPtr& causal_mask,
                                     const MemoryEfficientAttentionConfig& config) {
    if (!q || !k || !v || q->shape().size() != 4) throw TensorError("memory_efficient_attention: expects [B,heads,S,head_dim] tensors");
    const int64_t S = q->shape()[2], hd = q->shape()[3];
    const float scale = config.scale > 0.f ? config.scale : 1.0f / std::sqrt((float)hd);
    auto scores = mul(matmul(q, transpose(k, 2, 3)), scale);
    TensorPtr mask = causal_mask;
    if (!mask && config.use_causal_mask) mask = create_causal_mask((int)S);
    if (mask) scores = add(scores, mask);
    return matmul(softmax(scores, -1), v);
}

}  // namespace ops
