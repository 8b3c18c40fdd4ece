#include "auto_trainer.h"

#include <stdexcept>

namespace ops {

AutoTrainStepResult AutoTrainer::train_step(const TensorPtr& input_ids, const TensorPtr& attention_mask, const TensorPtr& labels) {
    if (config_.ignore_index != -100) throw std::runtime_error("AutoTrainer: ignore_index other than -100 is not supported by the device step");
    (void)attention_mask;     // all-ones masks only: padded batches are expressed through ignore_index labels
    const auto params = model_.trainable_parameters();
    if (params.empty()) throw std::runtime_error("AutoTrainer::train_step requires trainable parameters; call init_lora first");
    AutoTrainStepResult r;
    r.loss = model_.forward_backward(input_ids, labels);
    model_.optimizer_step(config_.learning_rate, 0.9f, 0.999f, 1e-8f, config_.weight_decay, config_.max_grad_norm, 0.0f);
    r.trainable_tensor_count = (int)params.size();
    return r;
}

}  // namespace ops
