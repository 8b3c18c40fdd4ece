// Causal-LM cross entropy (same functions as the reference's core/lm_loss.h).
#pragma once
#include <cmath>
#include <string>

#include "tensor.h"

namespace ops {

// logits [B,S,V] f32, labels [B,S] int32.  Row (b, s < S-1) is scored against labels[b, s+1];
// labels equal to ignore_index are skipped; "mean" divides by the number of scored rows (NaN if none).
TensorPtr lm_cross_entropy(const TensorPtr& logits, const TensorPtr& labels, int ignore_index = -100, const std::string& reduction = "mean");
// Same objective from hidden [B,S,H] and the lm-head weight [V,H] (f32, or frozen bf16/f16).
TensorPtr selected_token_lm_cross_entropy(const TensorPtr& hidden, const TensorPtr& lm_head_weight, const TensorPtr& labels,
                                          int ignore_index = -100, const std::string& reduction = "mean");
TensorPtr streaming_lm_cross_entropy(const TensorPtr& hidden, const TensorPtr& lm_head_weight, const TensorPtr& labels,
                                     int ignore_index = -100, const std::string& reduction = "mean");
inline float perplexity_from_loss(float mean_nll) { return std::exp(mean_nll); }

}  // namespace ops
