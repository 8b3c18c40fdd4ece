// Optimizer base (same interface as the reference's optim/optimizer.h).
#pragma once
#include <string>
#include <vector>

#include "../core/tensor.h"

namespace ops {

struct OptimizerConfig {
    float learning_rate;
    float weight_decay;
    float clip_grad_norm;
    bool amsgrad;
    OptimizerConfig(float lr = 1e-3f, float wd = 0.0f, float clip = 1.0f, bool ams = false)
        : learning_rate(lr), weight_decay(wd), clip_grad_norm(clip), amsgrad(ams) {}
    virtual ~OptimizerConfig() = default;
};

struct OptimizerState {
    virtual ~OptimizerState() = default;
    virtual void to_file(const std::string&) const {}
    virtual void from_file(const std::string&) {}
};

class Optimizer {
public:
    explicit Optimizer(const OptimizerConfig& config) : config_(config) {}
    virtual ~Optimizer() = default;
    virtual void step(const std::vector<TensorPtr>& parameters, const std::vector<TensorPtr>& gradients) = 0;
    virtual void save_state(const std::string& path) const = 0;
    virtual void load_state(const std::string& path) = 0;
    virtual void set_learning_rate(float lr) { config_.learning_rate = lr; }
    virtual float get_learning_rate() const { return config_.learning_rate; }
    void zero_grad(const std::vector<TensorPtr>& parameters) { for (auto& p : parameters) if (p) p->zero_grad(); }
    // scales every gradient by max_norm / ||g|| when the global L2 norm exceeds max_norm
    void clip_grad_norm(const std::vector<TensorPtr>& parameters, float max_norm);
    float compute_grad_norm(const std::vector<TensorPtr>& parameters);
    void scale_gradients(const std::vector<TensorPtr>& parameters, float scale);
protected:
    virtual void update_param(TensorPtr, const TensorPtr&, OptimizerState&) {}
    OptimizerConfig config_;
};

}  // namespace ops
