// AutoTrainer of the operator API (same interface as the reference's optim/auto_trainer.h): one call =
// forward -> lm_cross_entropy -> backward -> clip_grad_norm -> Adam::step -> zero_grad.  With a model of graph/*.h the
// forward / loss / backward part is one fused device pass and the adapters, their gradients and the Adam moments
// never leave the GPU.
#pragma once
#include <memory>

#include "../core/tensor.h"
#include "../graph/auto_model.h"
#include "adam.h"

namespace ops {

struct AutoTrainerConfig {            // field order as in the reference (aggregate initialisation)
    float learning_rate = 2e-4f, weight_decay = 0.0f;
    float max_grad_norm = 1.0f;       // <= 0: no clipping
    int ignore_index = -100;          // label value that is not scored
};

struct AutoTrainStepResult { float loss = 0.0f; int trainable_tensor_count = 0; };

class AutoTrainer {
    AutoModelForCausalLM& model_;
    AutoTrainerConfig config_;
    std::unique_ptr<Adam> optimizer_;     // created on the first step, over model_.trainable_parameters()
public:
    AutoTrainer(AutoModelForCausalLM& model, const AutoTrainerConfig& config = AutoTrainerConfig());
    // ids / mask / labels: int32 [B, S]; the mask may be null or right-padded
    AutoTrainStepResult train_step(const TensorPtr& input_ids, const TensorPtr& attention_mask, const TensorPtr& labels);
};

}  // namespace ops
