// Model family detection from a model directory's config.json (same types as the reference's graph/model_registry.h).
#pragma once
#include <string>
#include <vector>

namespace ops {

enum class ModelFamily { GPT2, Gemma, Qwen, Unknown };
std::string to_string(ModelFamily family);

struct ModelAssetPaths {
    std::string model_dir;
    std::string config_json_path;
};

struct ModelArchitectureSpec {
    ModelFamily family = ModelFamily::Unknown;
    std::string model_type;
    ModelAssetPaths assets;
    std::vector<std::string> default_lora_targets;
    bool tie_word_embeddings = false;
};

class ModelRegistry {
public:
    static ModelArchitectureSpec inspect_pretrained(const std::string& model_dir);
    static ModelFamily infer_family(const std::string& model_dir);
};

}  // namespace ops
