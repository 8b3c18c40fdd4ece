// LoRA injection for GPT-2 (the class surface of the reference's graph/lora_injector.h): creates A/B pairs and
// attaches them to the model's LoRALinear modules.
#pragma once
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/tensor.h"
#include "gpt2_model.h"

namespace ops {

enum class LoraTarget { AttnQKV, AttnProj, MlpFcIn, MlpFcOut };

struct LoraSpec {
    int rank = 8;
    float alpha = 16.0f;
    float dropout = 0.05f;             // stored in adapter files; the forward pass never applies it
    bool split_qkv = true;             // three [C,C] adapters on the q / k / v column ranges instead of one on [C,3C]
    std::vector<LoraTarget> targets = {LoraTarget::AttnQKV, LoraTarget::AttnProj};
    std::vector<int> layers;           // empty = all layers
    LoraSpec() = default;
    static LoraSpec default_config() { return LoraSpec(); }
    static LoraSpec full_config() {
        LoraSpec s;
        s.targets = {LoraTarget::AttnQKV, LoraTarget::AttnProj, LoraTarget::MlpFcIn, LoraTarget::MlpFcOut};
        return s;
    }
};

struct LoraState {
    TensorPtr A;          // [in, r]
    TensorPtr B;          // [r, out]
    float scale = 1.0f;   // alpha / r
    float dropout_p = 0.0f;
    bool enabled = true;
    void init(int64_t in_features, int64_t out_features, int rank, float alpha, float dropout);   // A ~ N(0, 1/r), B = 0
};

class LoraInjector {
public:
    LoraInjector() = default;
    ~LoraInjector() = default;

    void inject(GPT2Model& model, const LoraSpec& spec);
    void merge();
    void unmerge();
    void merge_all(GPT2Model& model);
    void unmerge_all(GPT2Model& model);
    std::vector<TensorPtr> collect_lora_parameters() const;
    void save_lora_safetensors(const std::string& path) const;
    void load_lora_safetensors(const std::string& path);
    void print_info() const;
    std::vector<TensorPtr> get_trainable_params();
    const LoraSpec& spec() const { return spec_; }
    // y = x W (+ bias) + scale (x A) B for a free-standing adapter state
    static TensorPtr lora_linear_forward(const TensorPtr& x, const TensorPtr& W, const TensorPtr& bias, const LoraState* lora, bool training = false);

private:
    LoraSpec spec_;
    bool merged_ = false;
    int num_layers_ = 0;
    GPT2Model* model_ = nullptr;
};

}  // namespace ops
