// AutoModelForCausalLM of the operator API (same entry points as the reference's graph/auto_model.h) on top of
// the device step engine (include/mft_step.h).  parameters() / trainable_parameters() hand out host-visible fp32
// tensors in the reference's order and layouts; the engine holds the device-resident copy (bf16 frozen weights,
// fp32 LoRA buckets) that the fused forward / backward kernels use.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../../../../include/mft_step.h"
#include "../core/tensor.h"
#include "model_registry.h"

namespace ops {

struct AutoModelLoadOptions {
    bool load_weights = true;     // SafeTensors ingest is outside the step's path: only load_weights = false is served here
    bool verbose = false;
};

struct AutoLoraConfig {
    int rank = 8;
    float alpha = 16.0f;
    float dropout = 0.05f;        // never applied by LoRALinear::forward in the reference either
    uint64_t seed = 42;
    std::vector<std::string> target_modules;
    static AutoLoraConfig attention_qkvo() {
        AutoLoraConfig c;
        c.target_modules = {"q_proj", "k_proj", "v_proj", "o_proj"};
        return c;
    }
};

class AutoModelForCausalLM {
public:
    static std::unique_ptr<AutoModelForCausalLM> from_pretrained(const std::string& model_dir, const AutoModelLoadOptions& options = AutoModelLoadOptions());
    ~AutoModelForCausalLM();

    void init_lora(const AutoLoraConfig& config = AutoLoraConfig());
    std::vector<TensorPtr> parameters();
    std::vector<TensorPtr> trainable_parameters();      // brings the host copies up to date with the device first
    ModelFamily family() const { return spec_.family; }
    const ModelArchitectureSpec& spec() const { return spec_; }
    const std::string& model_dir() const { return model_dir_; }
    const mft_model_config_t& config() const { return cfg_; }

    // Tell the model that parameters() / trainable_parameters() tensors were modified on the host since the last step.
    void mark_parameters_dirty() { params_dirty_ = true; }
    void mark_lora_dirty() { lora_dirty_ = true; }

    // One forward + lm_cross_entropy + backward on the device; gradients accumulate.  Returns the mean loss.
    float forward_backward(const TensorPtr& input_ids, const TensorPtr& labels);
    float forward_loss(const TensorPtr& input_ids, const TensorPtr& labels);
    void optimizer_step(float lr, float beta1, float beta2, float eps, float weight_decay, float max_grad_norm, float clip_eps = 0.0f);
    std::vector<TensorPtr> lora_gradients();            // host copies (nullptr where the reference delivers none)

private:
    AutoModelForCausalLM(std::string dir, ModelArchitectureSpec spec) : model_dir_(std::move(dir)), spec_(std::move(spec)) {}
    void ensure_engine(int batch, int seq);
    void sync_lora_to_host();

    std::string model_dir_;
    ModelArchitectureSpec spec_;
    mft_model_config_t cfg_{};
    mft_model_t* engine_ = nullptr;
    std::vector<TensorPtr> params_, lora_;
    bool params_dirty_ = true, lora_dirty_ = true, lora_host_stale_ = false;
};

}  // namespace ops
