// Qwen2 / Qwen2.5 decoder with LoRA on the attention projections: the class surface of the reference's
// graph/qwen_model.h, with forward() / forward_hidden() served by the device step engine (see engine_model.h).
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/tensor.h"
#include "../nn/lora_linear.h"

namespace ops {

namespace detail { class EngineModel; }

struct QwenConfig {                    // defaults: Qwen2.5-0.5B; names are config.json's
    int vocab_size = 151936, hidden_size = 896, intermediate_size = 4864;
    int num_hidden_layers = 24, num_attention_heads = 14, num_key_value_heads = 2;
    int max_position_embeddings = 32768;
    float rms_norm_eps = 1e-6f, rope_theta = 1000000.0f;
    std::string hidden_act = "silu";
    int bos_token_id = -1, eos_token_id = -1, pad_token_id = -1;
    static QwenConfig from_pretrained(const std::string& config_path);     // reads a config.json
};

struct QwenBlock {
    TensorPtr input_norm_weight, post_norm_weight;
    TensorPtr q_proj_weight, q_proj_bias;
    TensorPtr k_proj_weight, k_proj_bias;
    TensorPtr v_proj_weight, v_proj_bias;
    TensorPtr o_proj_weight;
    TensorPtr gate_proj_weight, up_proj_weight, down_proj_weight;
    std::unique_ptr<LoRALinear> q_lin, k_lin, v_lin, o_lin;
    bool lora_initialized = false;
};

class QwenModel {
public:
    explicit QwenModel(const QwenConfig& cfg);
    ~QwenModel();
    QwenModel(const QwenModel&) = delete;
    QwenModel& operator=(const QwenModel&) = delete;

    const QwenConfig& config() const { return config_; }
    const TensorPtr& embedding_weight() const { return embed_tokens_; }
    void assign_weight(const std::string& key, const TensorPtr& tensor);      // key: the reference's internal name
    void freeze_base();
    std::vector<TensorPtr> parameters() const;               // embed, final norm, 12 tensors per layer

    // A ~ U(-0.01, 0.01) from mt19937(seed), B = 0, on q and v (qv_only) or q, k, v, o.
    void init_lora(int rank = 8, float alpha = 16.0f, float dropout = 0.05f, bool qv_only = false, uint64_t seed = 42);
    std::vector<TensorPtr> get_lora_parameters() const;      // per layer: q, v, k, o (A then B)

    // all three are deferred values served by the device step engine
    TensorPtr forward(const TensorPtr& input_ids, const TensorPtr& attention_mask = nullptr);           // logits [B,S,V]
    TensorPtr forward_hidden(const TensorPtr& input_ids, const TensorPtr& attention_mask = nullptr);    // [B,S,hidden] after the final norm
    TensorPtr lm_head(const TensorPtr& hidden);                                                            // hidden . embed^T

private:
    QwenConfig config_;
    TensorPtr embed_tokens_, final_norm_weight_;
    std::vector<QwenBlock> layers_;
    std::shared_ptr<detail::EngineModel> impl_;
    void ensure_modules(QwenBlock& b);
};

}  // namespace ops
