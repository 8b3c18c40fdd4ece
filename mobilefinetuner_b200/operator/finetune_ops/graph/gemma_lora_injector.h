// LoRA injection for Gemma (the class surface of the reference's graph/gemma_lora_injector.h).  Adapter tensors use
// the PEFT layout: A [rank, in], B [out, rank].
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "gemma_model.h"

namespace ops {

struct GemmaLoraSpec {
    int rank = 8; float alpha = 32.0f;
    float dropout = 0.1f;              // stored in adapter files; the forward pass never applies it
    std::vector<std::string> target_modules = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"};
    std::vector<int> layers;           // empty = all layers
    // the three presets of the reference: all seven linears / the four attention projections / q and v only
    static GemmaLoraSpec with_targets(std::vector<std::string> t) { GemmaLoraSpec s; s.target_modules = std::move(t); return s; }
    static GemmaLoraSpec full_attn_mlp() { return GemmaLoraSpec(); }
    static GemmaLoraSpec attention_only() { return with_targets({"q_proj", "k_proj", "v_proj", "o_proj"}); }
    static GemmaLoraSpec attention_light() { return with_targets({"q_proj", "v_proj"}); }
};

class GemmaLoraInjector {
    GemmaModel* model_ = nullptr;      // the model of the last inject()
    GemmaLoraSpec spec_;
    int num_layers_ = 0, attached_modules_ = 0;
public:
    void inject(GemmaModel& model, const GemmaLoraSpec& spec);
    std::vector<TensorPtr> get_trainable_params() const;      // A then B per adapted linear, layer by layer
    // adapter files: keys "layer.{i}.{attn.q|attn.k|attn.v|attn.proj|mlp.gate|mlp.up|mlp.down}.lora_{A|B}", F32, sorted
    void load_lora_safetensors(const std::string& path);
    void save_lora_safetensors(const std::string& path) const;
    // W += scale * B A on the device weights and back (byte-exact restore)
    void merge_all(GemmaModel& model);
    void unmerge_all(GemmaModel& model);
    void print_info() const;
};

}  // namespace ops
