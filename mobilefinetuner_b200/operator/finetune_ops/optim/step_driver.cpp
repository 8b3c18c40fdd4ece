#include "step_driver.h"

#include <algorithm>
#include <cmath>

#include "../core/autograd_engine.h"
#include "../core/lm_loss.h"
#include "../core/memory_manager.h"
#include "../core/ops.h"

namespace ops {
namespace detail {

StepDriver::StepDriver(Forward f, Params p, const AdamConfig& adam, const StepDriverConfig& cfg)
    : forward_(std::move(f)), params_(std::move(p)), optimizer_(std::make_unique<Adam>(adam)), cfg_(cfg) {}

float StepDriver::lr_at(int step, int64_t num_sequences) const {
    const int64_t micro_per_epoch = (num_sequences + cfg_.micro_batch_size - 1) / cfg_.micro_batch_size;
    int64_t total = (micro_per_epoch * cfg_.num_epochs + cfg_.grad_accum_steps - 1) / cfg_.grad_accum_steps;
    total = std::max<int64_t>(1, total);
    const int warmup = static_cast<int>(total * cfg_.warmup_ratio);
    if (warmup > 0 && step <= warmup) return cfg_.learning_rate * (static_cast<float>(step) / warmup);
    float progress = static_cast<float>(step - warmup) / std::max<int64_t>(1, total - warmup);
    progress = std::clamp(progress, 0.0f, 1.0f);
    if (cfg_.lr_scheduler == "cosine") return cfg_.learning_rate * 0.5f * (1.0f + std::cos(3.14159265f * progress));
    if (cfg_.lr_scheduler == "linear" || !cfg_.constant_when_unknown) return cfg_.learning_rate * (1.0f - progress);
    return cfg_.learning_rate;
}

// scale = max / (norm + 1e-6) when norm > max (optim/trainer.cpp:75-99, optim/gemma_trainer.cpp:62-83), on the device
void StepDriver::clip(const std::vector<TensorPtr>& params) {
    const float norm = optimizer_->compute_grad_norm(params);
    if (norm > cfg_.max_grad_norm) optimizer_->scale_gradients(params, cfg_.max_grad_norm / (norm + 1e-6f));
}

float StepDriver::micro_step(const TensorPtr& ids, const TensorPtr& mask, const TensorPtr& labels, int64_t num_sequences) {
    auto loss = lm_cross_entropy(forward_(ids, mask), labels, -100, "mean");
    const float loss_val = static_cast<const Tensor&>(*loss).data<float>()[0];
    mul(loss, 1.0f / static_cast<float>(cfg_.grad_accum_steps))->backward();
    accum_counter_++;
    accum_loss_ += loss_val;
    if (accum_counter_ < cfg_.grad_accum_steps) return -1.0f;
    const auto params = params_();
    clip(params);
    std::vector<TensorPtr> grads;
    grads.reserve(params.size());
    for (const auto& p : params) grads.push_back(p->grad());
    global_step_++;
    optimizer_->set_learning_rate(lr_at(global_step_, num_sequences));
    optimizer_->step(params, grads);
    for (const auto& p : params)
        if (p->grad()) p->zero_grad();
    MemoryManager::instance().force_cleanup();
    accum_counter_ = 0;
    const float avg = accum_loss_ / static_cast<float>(cfg_.grad_accum_steps);
    accum_loss_ = 0.0f;
    return avg;
}

float StepDriver::eval_loss(const TensorPtr& ids, const TensorPtr& mask, const TensorPtr& labels) {
    autograd::NoGradGuard no_grad;                 // forward + loss only
    auto loss = lm_cross_entropy(forward_(ids, mask), labels, -100, "mean");
    return static_cast<const Tensor&>(*loss).data<float>()[0];
}

}  // namespace detail
}  // namespace ops
