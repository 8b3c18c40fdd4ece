#include "model_registry.h"

#include <algorithm>
#include <cctype>
#include <filesystem>
#include <stdexcept>

#include "json_fields.h"

namespace ops {

std::string to_string(ModelFamily f) {
    switch (f) {
        case ModelFamily::GPT2: return "gpt2";
        case ModelFamily::Gemma: return "gemma";
        case ModelFamily::Qwen: return "qwen";
        default: return "unknown";
    }
}

ModelFamily ModelRegistry::infer_family(const std::string& dir) { return inspect_pretrained(dir).family; }

ModelArchitectureSpec ModelRegistry::inspect_pretrained(const std::string& dir) {
    namespace fs = std::filesystem;
    const fs::path root(dir);
    std::error_code ec;
    if (!fs::exists(root / "config.json", ec)) throw std::runtime_error("Model directory is missing config.json: " + dir);
    const std::string js = detail::read_config_text((root / "config.json").string());
    ModelArchitectureSpec s;
    s.model_type = detail::json_string(js, "model_type", "");
    std::string t = s.model_type;
    std::transform(t.begin(), t.end(), t.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (t.find("qwen") != std::string::npos) { s.family = ModelFamily::Qwen; s.default_lora_targets = {"q_proj", "k_proj", "v_proj", "o_proj"}; }
    else if (t.find("gemma") != std::string::npos) { s.family = ModelFamily::Gemma; s.default_lora_targets = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"}; }
    else if (t.find("gpt2") != std::string::npos || t.find("gpt_2") != std::string::npos || t == "gpt") { s.family = ModelFamily::GPT2; s.default_lora_targets = {"attn_qkv", "attn_proj"}; }
    else throw std::runtime_error("Unsupported model_type in config.json: " + s.model_type);
    s.tie_word_embeddings = detail::json_bool(js, "tie_word_embeddings", s.family == ModelFamily::GPT2);
    ModelAssetPaths& a = s.assets;
    a.model_dir = dir;
    a.config_json_path = (root / "config.json").string();
    a.tokenizer_json_path = (root / "tokenizer.json").string();
    a.vocab_json_path = (root / "vocab.json").string();
    a.merges_txt_path = (root / "merges.txt").string();
    a.safetensors_path = (root / "model.safetensors").string();
    a.safetensors_index_path = (root / "model.safetensors.index.json").string();
    a.has_tokenizer_json = fs::exists(a.tokenizer_json_path, ec);
    a.has_vocab_json = fs::exists(a.vocab_json_path, ec);
    a.has_merges_txt = fs::exists(a.merges_txt_path, ec);
    a.has_single_safetensors = fs::exists(a.safetensors_path, ec);
    a.has_sharded_safetensors = fs::exists(a.safetensors_index_path, ec);
    return s;
}

}  // namespace ops
