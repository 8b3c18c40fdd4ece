// Adam optimizer (same interface as the reference's optim/adam.h): L2-style weight decay folded into the
// gradient, bias corrections 1 - pow(beta, step), epsilon added outside the square root.  The update of every
// parameter tensor is one kernel launch on its device copy; moments live on the device.
#pragma once
#include <unordered_map>

#include "optimizer.h"

namespace ops {

struct AdamConfig : public OptimizerConfig {
    float beta1, beta2, epsilon;
    AdamConfig() : OptimizerConfig(), beta1(0.9f), beta2(0.999f), epsilon(1e-8f) {}
    AdamConfig(float lr, float b1 = 0.9f, float b2 = 0.999f, float eps = 1e-8f, float wd = 0.0f, float clip = 1.0f, bool ams = false)
        : OptimizerConfig(lr, wd, clip, ams), beta1(b1), beta2(b2), epsilon(eps) {}
};

struct AdamState : public OptimizerState {
    size_t step = 0;
    std::vector<TensorPtr> m, v, v_hat;
};

class Adam : public Optimizer {
public:
    explicit Adam(const AdamConfig& config) : Optimizer(config), adam_config_(config) {}
    void step(const std::vector<TensorPtr>& parameters, const std::vector<TensorPtr>& gradients) override;
    void save_state(const std::string& path) const override;
    void load_state(const std::string& path) override;
    void set_learning_rate(float lr) override { adam_config_.learning_rate = lr; }
    float get_learning_rate() const override { return adam_config_.learning_rate; }
private:
    AdamConfig adam_config_;
    std::unordered_map<TensorPtr, AdamState> states_;
};

}  // namespace ops
