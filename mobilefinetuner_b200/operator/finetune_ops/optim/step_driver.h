// The body the two trainers share: gradient accumulation over micro-batches, the trainers' clip rule, the warm-up +
// linear / cosine learning-rate schedule and the Adam step, written over the public operator API.  With the models of
// graph/*.h every piece runs on the device (the adapters, their gradients and the Adam moments stay there); per window
// the host reads one scalar per micro-batch (the loss) and one for the gradient norm.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../core/tensor.h"
#include "adam.h"

namespace ops {
namespace detail {

struct StepDriverConfig {
    float learning_rate = 2e-4f, max_grad_norm = 1.0f, warmup_ratio = 0.03f;
    std::string lr_scheduler = "linear";          // "linear", "cosine", anything else: constant
    bool constant_when_unknown = true;             // LoRATrainer keeps the base rate for an unknown scheduler, GemmaLoRATrainer decays linearly
    int grad_accum_steps = 1, micro_batch_size = 1, num_epochs = 1;
};

class StepDriver {
public:
    using Forward = std::function<TensorPtr(const TensorPtr& ids, const TensorPtr& mask)>;
    using Params = std::function<std::vector<TensorPtr>()>;
    StepDriver(Forward forward, Params params, const AdamConfig& adam, const StepDriverConfig& cfg);

    // get_lr of the trainers (optim/trainer.cpp:50-73, optim/gemma_trainer.cpp:44-60): integer / float arithmetic kept
    float lr_at(int step, int64_t num_sequences) const;
    // One micro-batch.  Returns the window's mean loss when this call closed an accumulation window, else -1.
    // lr_step_offset: LoRATrainer takes the rate of step + 1 before it counts the step, GemmaLoRATrainer counts first.
    float micro_step(const TensorPtr& ids, const TensorPtr& mask, const TensorPtr& labels, int64_t num_sequences);
    float eval_loss(const TensorPtr& ids, const TensorPtr& mask, const TensorPtr& labels);
    int global_step() const { return global_step_; }

private:
    Forward forward_;
    Params params_;
    std::unique_ptr<Adam> optimizer_;
    StepDriverConfig cfg_;
    int global_step_ = 0, accum_counter_ = 0;
    float accum_loss_ = 0.0f;
    void clip(const std::vector<TensorPtr>& params);
};

}  // namespace detail
}  // namespace ops
