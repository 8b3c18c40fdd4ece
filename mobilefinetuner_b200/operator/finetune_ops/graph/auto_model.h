// AutoModelForCausalLM of the operator API (same entry points as the reference's graph/auto_model.h): picks the model
// class from config.json, optionally loads a SafeTensors snapshot, injects LoRA, forwards.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../core/tensor.h"
#include "gemma_lora_injector.h"
#include "gemma_model.h"
#include "gpt2_model.h"
#include "lora_injector.h"
#include "model_registry.h"
#include "qwen_model.h"
#include "safetensors_loader.h"

namespace ops {

struct AutoModelLoadOptions {
    bool load_weights = true, verbose = false;    // load_weights: read the snapshot's *.safetensors into the model
    SafeTensorsLoadOptions safetensors_options;
    AutoModelLoadOptions() { safetensors_options.verbose = false; }
};

struct AutoLoraConfig {
    int rank = 8; float alpha = 16.0f;
    float dropout = 0.05f;        // never applied by LoRALinear::forward in the reference either
    uint64_t seed = 42;           // of the adapters' initial values
    // GPT-2: "c_attn" / "attn_qkv" select ONE adapter on the fused [C,3C] projection; "q_proj" / "k_proj" / "v_proj"
    // (and the default, an empty list) select three adapters on its column ranges, which - as in the reference - only
    // add to the forward value and never receive a gradient.
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

    // logits [B, S, V] as a deferred value: lm_cross_entropy on it runs the fused step, reading it materialises it
    TensorPtr forward(const TensorPtr& input_ids, const TensorPtr& attention_mask = nullptr);
    void init_lora(const AutoLoraConfig& config = AutoLoraConfig());
    std::vector<TensorPtr> parameters();              // frozen weights in the model class's own order
    std::vector<TensorPtr> trainable_parameters();    // A then B per adapted linear
    // exactly one of the three is non-null
    GPT2Model* gpt2() { return gpt2_.get(); }
    QwenModel* qwen() { return qwen_.get(); }
    GemmaModel* gemma() { return gemma_.get(); }
    const ModelArchitectureSpec& spec() const { return spec_; }
    ModelFamily family() const { return spec_.family; }
    const std::string& model_dir() const { return model_dir_; }

private:
    AutoModelForCausalLM(std::string dir, ModelArchitectureSpec spec) : model_dir_(std::move(dir)), spec_(std::move(spec)) {}
    void load_pretrained_weights(const AutoModelLoadOptions& options);

    std::string model_dir_;
    ModelArchitectureSpec spec_;
    std::unique_ptr<GPT2Model> gpt2_; std::unique_ptr<LoraInjector> gpt2_lora_;
    std::unique_ptr<GemmaModel> gemma_; std::unique_ptr<GemmaLoraInjector> gemma_lora_;
    std::unique_ptr<QwenModel> qwen_;
};

}  // namespace ops
