// What a pretrained model directory holds: the model family named by config.json and which tokenizer / weight files
// sit next to it (same types as the reference's graph/model_registry.h).
#pragma once
#include <string>
#include <vector>

namespace ops {

enum class ModelFamily { GPT2, Gemma, Qwen, Unknown };
std::string to_string(ModelFamily family);

struct ModelAssetPaths {
    std::string model_dir, config_json_path;
    std::string tokenizer_json_path, vocab_json_path, merges_txt_path;
    std::string safetensors_path, safetensors_index_path;
    bool has_tokenizer_json = false, has_vocab_json = false, has_merges_txt = false;
    bool has_single_safetensors = false, has_sharded_safetensors = false;
};

struct ModelArchitectureSpec {
    ModelFamily family = ModelFamily::Unknown;
    std::string model_type;                           // config.json "model_type" as written
    ModelAssetPaths assets;
    std::vector<std::string> default_lora_targets;    // HuggingFace module names the family's CLIs adapt by default
    bool tie_word_embeddings = false;
};

class ModelRegistry {
public:
    static ModelFamily infer_family(const std::string& model_dir);
    // throws without a config.json or for an unknown model_type
    static ModelArchitectureSpec inspect_pretrained(const std::string& model_dir);
};

}  // namespace ops
