// LoRA injection for Gemma (the class surface of the reference's graph/gemma_lora_injector.h).  Adapter tensors use
// the PEFT layout: A [rank, in], B [out, rank].
#pragma once
#include <string>
#include <vector>

#include "gemma_model.h"

namespace ops {

struct GemmaLoraSpec {
    int rank = 8;
    float alpha = 32.0f;
    float dropout = 0.1f;              // stored in adapter files; the forward pass never applies it
    std::vector<std::string> target_modules = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"};
    std::vector<int> layers;           // empty = all layers
    static GemmaLoraSpec full_attn_mlp() { return GemmaLoraSpec(); }
    static GemmaLoraSpec attention_only() {
        GemmaLoraSpec s;
        s.target_modules = {"q_proj", "k_proj", "v_proj", "o_proj"};
        return s;
    }
    static GemmaLoraSpec attention_light() {
        GemmaLoraSpec s;
        s.target_modules = {"q_proj", "v_proj"};
        return s;
    }
};

class GemmaLoraInjector {
public:
    GemmaLoraInjector() = default;
    ~GemmaLoraInjector() = default;

    void inject(GemmaModel& model, const GemmaLoraSpec& spec);
    std::vector<TensorPtr> get_trainable_params() const;
    void print_info() const;
    // keys "layer.{i}.{attn.q|attn.k|attn.v|attn.proj|mlp.gate|mlp.up|mlp.down}.lora_{A|B}", F32, sorted
    void save_lora_safetensors(const std::string& path) const;
    void load_lora_safetensors(const std::string& path);
    void merge_all(GemmaModel& model);
    void unmerge_all(GemmaModel& model);

private:
    GemmaModel* model_ = nullptr;
    GemmaLoraSpec spec_;
    int num_layers_ = 0;
    int attached_modules_ = 0;
};

}  // namespace ops
