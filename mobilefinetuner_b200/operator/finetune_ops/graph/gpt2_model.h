// GPT-2 with LoRA-ready linears: the class surface of the reference's graph/gpt2_model.h (configuration, per-block
// weight tensors and LoRALinear modules, assign_weight, parameters() order), with forward() served by the device
// step engine instead of a layer-by-layer operator graph (see engine_model.h).
#pragma once
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../core/tensor.h"
#include "../nn/lora_linear.h"

namespace ops {

namespace detail { class EngineModel; }

struct GPT2BlockWeights {
    TensorPtr ln_1_weight, ln_1_bias;
    TensorPtr ln_2_weight, ln_2_bias;
    TensorPtr attn_qkv_weight, attn_qkv_bias;        // [C, 3C], [3C]
    TensorPtr attn_proj_weight, attn_proj_bias;      // [C, C], [C]
    TensorPtr mlp_fc_in_weight, mlp_fc_in_bias;      // [C, 4C], [4C]
    TensorPtr mlp_fc_out_weight, mlp_fc_out_bias;    // [4C, C], [C]
    std::unique_ptr<LoRALinear> qkv_lin, proj_lin, fc_in_lin, fc_out_lin;
    bool lora_initialized = false;
};

struct GPT2Config {
    int vocab_size = 50257;
    int n_positions = 1024;
    int n_embd = 768;
    int n_layer = 12;
    int n_head = 12;
    float layernorm_eps = 1e-5f;
    bool tie_word_embeddings = true;
    bool use_cache = false;
    bool use_memory_efficient_attention = true;      // the device attention kernels never materialise the scores either way
    bool use_bf16_activations = false;               // device activations are bf16 regardless
    static GPT2Config from_pretrained(const std::string& config_path_or_dir);
};

class GPT2Model {
public:
    explicit GPT2Model(const GPT2Config& config);
    ~GPT2Model();
    GPT2Model(const GPT2Model&) = delete;
    GPT2Model& operator=(const GPT2Model&) = delete;

    // input_ids int32 [B,S] -> logits [B,S,vocab] (deferred: lm_cross_entropy consumes them without forming them)
    TensorPtr forward(const TensorPtr& input_ids, const TensorPtr& attention_mask = nullptr);
    void tie_weights();
    void assign_weight(const std::string& key, const TensorPtr& tensor);
    std::vector<TensorPtr> parameters();             // wte, wpe, 12 tensors per block, ln_f weight and bias
    std::vector<TensorPtr> trainable_parameters();
    void freeze_base_parameters();
    void print_model_info() const;
    const GPT2Config& config() const { return config_; }

    std::pair<TensorPtr*, TensorPtr*> attn_qkv_params(int i);
    std::pair<TensorPtr*, TensorPtr*> attn_proj_params(int i);
    std::pair<TensorPtr*, TensorPtr*> mlp_fc_in_params(int i);
    std::pair<TensorPtr*, TensorPtr*> mlp_fc_out_params(int i);
    GPT2BlockWeights& get_block(int i) { return blocks_[(size_t)i]; }
    const GPT2BlockWeights& get_block(int i) const { return blocks_[(size_t)i]; }
    std::vector<TensorPtr> get_lora_parameters();
    void init_lora_modules();

private:
    GPT2Config config_;
    TensorPtr wte_weight_, wpe_weight_;
    std::vector<GPT2BlockWeights> blocks_;
    TensorPtr ln_f_weight_, ln_f_bias_;
    bool weights_tied_ = false;
    std::shared_ptr<detail::EngineModel> impl_;
    GPT2BlockWeights& block_at(int i, const char* who);
};

}  // namespace ops
