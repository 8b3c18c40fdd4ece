// Adapter files for GPT-2 (the class surface of the reference's graph/lora_saver.h): keys
// "layer.{i}.{attn.qkv|attn.q|attn.k|attn.v|attn.proj|mlp.fc_in|mlp.fc_out}.lora_{A|B}", F32, sorted, with rank / alpha /
// dropout / split_qkv / targets in the container's metadata.
#pragma once
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/tensor.h"
#include "gpt2_model.h"
#include "lora_injector.h"

namespace ops {

struct LoRAState {                    // what an adapter file holds
    int rank = 8; float alpha = 16.0f, dropout = 0.0f;
    bool split_qkv = true;            // q / k / v adapters (true) or one fused qkv adapter
    std::vector<LoraTarget> targets;
    std::unordered_map<std::string, TensorPtr> tensors;      // key -> f32 tensor as stored
    bool compatible_with(const GPT2Model& model) const;      // layer count and shapes fit the model
};

class LoraSaver {
public:
    // keys: "layer.<i>.<target>.lora_<A|B>"
    static std::string make_peft_key(int layer, const std::string& target, const std::string& ab);
    static bool parse_peft_key(const std::string& key, int& layer, std::string& target, std::string& ab);
    static LoRAState load_safetensors(const std::string& path);
    static void save_safetensors(const std::string& path, const GPT2Model& model, const LoraSpec& spec);
    static void attach_from_state(GPT2Model& model, const LoRAState& state);     // injects and fills the adapters
};

}  // namespace ops
