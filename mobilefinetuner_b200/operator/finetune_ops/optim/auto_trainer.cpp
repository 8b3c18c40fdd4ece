#include "auto_trainer.h"

#include <stdexcept>

#include "../core/lm_loss.h"

namespace ops {

AutoTrainer::AutoTrainer(AutoModelForCausalLM& model, const AutoTrainerConfig& config) : model_(model), config_(config) {
    AdamConfig a;
    a.learning_rate = config_.learning_rate;
    a.weight_decay = config_.weight_decay;
    a.clip_grad_norm = config_.max_grad_norm;
    optimizer_ = std::make_unique<Adam>(a);
}

AutoTrainStepResult AutoTrainer::train_step(const TensorPtr& input_ids, const TensorPtr& attention_mask, const TensorPtr& labels) {
    const auto params = model_.trainable_parameters();
    if (params.empty()) throw std::runtime_error("AutoTrainer::train_step requires trainable parameters; call init_lora first");
    auto loss = lm_cross_entropy(model_.forward(input_ids, attention_mask), labels, config_.ignore_index, "mean");
    loss->backward();
    optimizer_->clip_grad_norm(params, config_.max_grad_norm);
    std::vector<TensorPtr> grads;
    grads.reserve(params.size());
    for (const auto& p : params) grads.push_back(p->grad());
    optimizer_->step(params, grads);
    optimizer_->zero_grad(params);
    AutoTrainStepResult r;
    r.loss = static_cast<const Tensor&>(*loss).data<float>()[0];
    r.trainable_tensor_count = (int)params.size();
    return r;
}

}  // namespace ops
