// Gemma-3 text decoder (sliding + global attention, QK-norm, GeGLU, (1 + w) RMSNorm, tied lm head) with LoRA on any of
// its seven linears: the class surface of the reference's graph/gemma_model.h, with forward() served by the device
// step engine (see engine_model.h).  The reference's debugging hooks (tensor dumps, numeric perturbation) are kept
// as accepted no-ops: there are no per-layer host tensors to dump on this path.
#pragma once
#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../core/tensor.h"
#include "../nn/lora_linear.h"

namespace ops {

namespace detail { class EngineModel; }

struct GemmaTextConfig {                       // defaults: Gemma-3-270M; names are config.json's
    int vocab_size = 262144, hidden_size = 640, intermediate_size = 2048;
    int num_hidden_layers = 18, num_attention_heads = 4, num_key_value_heads = 1, head_dim = 256;
    int max_position_embeddings = 32768;
    int sliding_window = 512;                  // tokens a "sliding_attention" layer looks back
    bool attention_bias = false, use_bidirectional_attention = false, use_cache = true;
    float attention_dropout = 0.0f;
    float rms_norm_eps = 1e-6f;
    float query_pre_attn_scalar = 256.0f;      // attention scale = 1 / sqrt(this)
    float attn_logit_softcapping = 0.0f;       // parsed, never applied (as in the reference's graph)
    float final_logit_softcapping = 0.0f;
    float rope_theta = 1000000.0f, rope_local_base_freq = 10000.0f;      // global / sliding layers
    std::string hidden_activation = "gelu_pytorch_tanh";
    std::vector<std::string> layer_types;      // "sliding_attention" / "full_attention" per layer; empty = all sliding
    static GemmaTextConfig from_pretrained(const std::string& model_dir);
};

struct GemmaBlockWeights {
    TensorPtr input_layernorm_weight, post_attention_layernorm_weight;
    TensorPtr pre_feedforward_layernorm_weight, post_feedforward_layernorm_weight;
    TensorPtr q_proj_weight, k_proj_weight, v_proj_weight, o_proj_weight;      // [in, out]
    TensorPtr q_norm_weight, k_norm_weight;                                    // [head_dim]
    TensorPtr gate_proj_weight, up_proj_weight, down_proj_weight;
    std::unique_ptr<LoRALinear> q_proj_lora, k_proj_lora, v_proj_lora, o_proj_lora, gate_proj_lora, up_proj_lora, down_proj_lora;
    bool lora_initialized = false;
};

struct EmbeddingDumpRequest {
    bool active = false;
    int target_step = 0;
    std::string output_dir;
    bool fulfilled = false;
};

class GemmaModel {
public:
    explicit GemmaModel(const GemmaTextConfig& config);
    ~GemmaModel();
    GemmaModel(const GemmaModel&) = delete;
    GemmaModel& operator=(const GemmaModel&) = delete;

    TensorPtr forward(const TensorPtr& input_ids, const TensorPtr& attention_mask = nullptr);
    void assign_weight(const std::string& key, const TensorPtr& tensor);
    const GemmaTextConfig& config() const { return config_; }
    void init_lora_modules();
    GemmaBlockWeights& get_block(int i);
    const GemmaBlockWeights& get_block(int i) const;
    std::vector<TensorPtr> parameters() const;               // embed, final norm, lm head copy, 13 tensors per layer
    std::vector<TensorPtr> get_lora_parameters() const;      // per layer: q, k, v, o, gate, up, down (A then B)
    void merge_lora();
    void unmerge_lora();

    void request_embedding_dump(int step, const std::string& output_dir);
    void enable_debug_dump(const std::string& dir, const std::vector<int>& layers);
    void disable_debug_dump();
    bool debug_enabled() const { return debug_.enabled; }
    const std::unordered_map<std::string, TensorPtr>& debug_tensors() const { return debug_.tensors; }
    void set_debug_retain_grads(bool retain) { debug_.retain_grads = retain; }
    void set_numeric_perturb(bool enable, const std::string& name, int64_t index, float eps);
    void dump_layer_norm_weights(int layer, const std::string& dir) const;

private:
    GemmaTextConfig config_;
    TensorPtr embed_weight_, norm_weight_, lm_head_weight_;
    std::vector<GemmaBlockWeights> blocks_;
    bool lm_head_initialized_ = false;
    EmbeddingDumpRequest dump_request_;
    struct DebugConfig {
        bool enabled = false;
        std::string dir;
        std::unordered_set<int> layers;
        mutable std::unordered_map<std::string, TensorPtr> tensors;
        bool retain_grads = true;
    };
    mutable DebugConfig debug_;
    std::shared_ptr<detail::EngineModel> impl_;
};

}  // namespace ops
