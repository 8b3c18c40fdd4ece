#include "gemma_model.h"

#include <cmath>
#include <iostream>
#include <regex>
#include <stdexcept>

#include "../core/ops.h"
#include "engine_model.h"
#include "json_fields.h"

namespace ops {

GemmaTextConfig GemmaTextConfig::from_pretrained(const std::string& model_dir) {
    const std::string js = detail::read_config_text(model_dir);
    GemmaTextConfig c;
    c.vocab_size = detail::json_int(js, "vocab_size", c.vocab_size);
    c.hidden_size = detail::json_int(js, "hidden_size", c.hidden_size);
    c.intermediate_size = detail::json_int(js, "intermediate_size", c.intermediate_size);
    c.num_hidden_layers = detail::json_int(js, "num_hidden_layers", c.num_hidden_layers);
    c.num_attention_heads = detail::json_int(js, "num_attention_heads", c.num_attention_heads);
    c.num_key_value_heads = detail::json_int(js, "num_key_value_heads", c.num_key_value_heads);
    c.head_dim = detail::json_int(js, "head_dim", c.head_dim);
    c.max_position_embeddings = detail::json_int(js, "max_position_embeddings", c.max_position_embeddings);
    c.sliding_window = detail::json_int(js, "sliding_window", c.sliding_window);
    c.attention_bias = detail::json_bool(js, "attention_bias", c.attention_bias);
    c.use_bidirectional_attention = detail::json_bool(js, "use_bidirectional_attention", c.use_bidirectional_attention);
    c.use_cache = detail::json_bool(js, "use_cache", c.use_cache);
    c.attention_dropout = detail::json_float(js, "attention_dropout", c.attention_dropout);
    c.rms_norm_eps = detail::json_float(js, "rms_norm_eps", c.rms_norm_eps);
    c.query_pre_attn_scalar = detail::json_float(js, "query_pre_attn_scalar", c.query_pre_attn_scalar);
    c.attn_logit_softcapping = detail::json_float(js, "attn_logit_softcapping", c.attn_logit_softcapping);
    c.final_logit_softcapping = detail::json_float(js, "final_logit_softcapping", c.final_logit_softcapping);
    c.rope_theta = detail::json_float(js, "rope_theta", c.rope_theta);
    c.rope_local_base_freq = detail::json_float(js, "rope_local_base_freq", c.rope_local_base_freq);
    c.hidden_activation = detail::json_string(js, "hidden_activation", c.hidden_activation);
    c.layer_types = detail::json_string_array(js, "layer_types");
    if (c.layer_types.empty()) c.layer_types.assign((size_t)c.num_hidden_layers, "sliding_attention");
    return c;
}

static TensorPtr zeros_f32(std::vector<int64_t> shape) { return std::make_shared<Tensor>(shape, kFloat32, kCPU); }

// The engine describes the attention pattern as "every k-th layer is global".  layer_types must fit that form.
static int global_period(const GemmaTextConfig& c) {
    int first = -1;
    for (int i = 0; i < (int)c.layer_types.size() && i < c.num_hidden_layers; ++i)
        if (c.layer_types[(size_t)i] == "full_attention") { first = i; break; }
    if (first < 0) return 0;
    const int k = first + 1;
    for (int i = 0; i < c.num_hidden_layers; ++i) {
        const bool full = i < (int)c.layer_types.size() && c.layer_types[(size_t)i] == "full_attention";
        if (full != ((i + 1) % k == 0))
            throw std::runtime_error("GemmaModel: layer_types must place a full-attention layer at every k-th position (k = " + std::to_string(k) + ")");
    }
    return k;
}

GemmaModel::GemmaModel(const GemmaTextConfig& config) : config_(config) {
    if (config_.layer_types.empty()) config_.layer_types.assign((size_t)config_.num_hidden_layers, "sliding_attention");
    const int64_t H = config_.hidden_size, I = config_.intermediate_size, hd = config_.head_dim;
    const int64_t QD = config_.num_attention_heads * hd, KD = config_.num_key_value_heads * hd;
    embed_weight_ = zeros_f32({config_.vocab_size, H});
    norm_weight_ = zeros_f32({H});
    lm_head_weight_ = zeros_f32({H, config_.vocab_size});
    blocks_.resize((size_t)config_.num_hidden_layers);
    for (auto& b : blocks_) {
        b.input_layernorm_weight = zeros_f32({H}); b.post_attention_layernorm_weight = zeros_f32({H});
        b.pre_feedforward_layernorm_weight = zeros_f32({H}); b.post_feedforward_layernorm_weight = zeros_f32({H});
        b.q_proj_weight = zeros_f32({H, QD}); b.k_proj_weight = zeros_f32({H, KD}); b.v_proj_weight = zeros_f32({H, KD});
        b.o_proj_weight = zeros_f32({QD, H});
        b.q_norm_weight = zeros_f32({hd}); b.k_norm_weight = zeros_f32({hd});
        b.gate_proj_weight = zeros_f32({H, I}); b.up_proj_weight = zeros_f32({H, I}); b.down_proj_weight = zeros_f32({I, H});
    }
    mft_model_config_t a{};
    a.family = MFT_FAMILY_GEMMA;
    a.vocab = config_.vocab_size; a.hidden = config_.hidden_size; a.inter = config_.intermediate_size; a.layers = config_.num_hidden_layers;
    a.n_heads = config_.num_attention_heads; a.n_kv_heads = config_.num_key_value_heads; a.head_dim = config_.head_dim;
    a.norm_eps = config_.rms_norm_eps; a.rope_theta = config_.rope_theta; a.rope_local_theta = config_.rope_local_base_freq;
    a.attn_scale = std::pow(config_.query_pre_attn_scalar, -0.5f);
    a.sliding_window = config_.sliding_window;
    a.global_every = global_period(config_);
    a.gpt2_detach_attn = 1;
    impl_ = std::make_shared<detail::EngineModel>(
        a, [this] { return parameters(); },
        [this](int layer, uint32_t target) -> LoRALinear* {
            GemmaBlockWeights& b = blocks_[(size_t)layer];
            switch (target) {
                case MFT_LORA_Q: return b.q_proj_lora.get();
                case MFT_LORA_K: return b.k_proj_lora.get();
                case MFT_LORA_V: return b.v_proj_lora.get();
                case MFT_LORA_O: return b.o_proj_lora.get();
                case MFT_LORA_GATE: return b.gate_proj_lora.get();
                case MFT_LORA_UP: return b.up_proj_lora.get();
                case MFT_LORA_DOWN: return b.down_proj_lora.get();
                default: return nullptr;
            }
        });
}

GemmaModel::~GemmaModel() = default;

TensorPtr GemmaModel::forward(const TensorPtr& ids, const TensorPtr& mask) { return impl_->forward(ids, mask); }

void GemmaModel::assign_weight(const std::string& key, const TensorPtr& t) {
    if (key == "embed_tokens.weight") {
        embed_weight_ = t;
        if (!lm_head_initialized_) {              // the tied head is kept as a transposed copy, as the reference does
            lm_head_weight_ = transpose(t, 0, 1);
            lm_head_initialized_ = true;
        }
        return;
    }
    if (key == "norm.weight") { norm_weight_ = t; return; }
    if (key == "lm_head.weight") { lm_head_weight_ = t; lm_head_initialized_ = true; return; }
    std::smatch m;
    if (!std::regex_match(key, m, std::regex(R"(layers\.(\d+)\.(.+))"))) throw std::runtime_error("Unknown Gemma weight key: " + key);
    const int layer = std::stoi(m[1].str());
    if (layer < 0 || layer >= config_.num_hidden_layers) throw std::runtime_error("Invalid Gemma layer index: " + std::to_string(layer));
    GemmaBlockWeights& b = blocks_[(size_t)layer];
    const std::unordered_map<std::string, TensorPtr*> slots = {
        {"input_layernorm.weight", &b.input_layernorm_weight}, {"post_attention_layernorm.weight", &b.post_attention_layernorm_weight},
        {"pre_feedforward_layernorm.weight", &b.pre_feedforward_layernorm_weight},
        {"post_feedforward_layernorm.weight", &b.post_feedforward_layernorm_weight},
        {"self_attn.q_proj.weight", &b.q_proj_weight}, {"self_attn.k_proj.weight", &b.k_proj_weight},
        {"self_attn.v_proj.weight", &b.v_proj_weight}, {"self_attn.o_proj.weight", &b.o_proj_weight},
        {"self_attn.q_norm.weight", &b.q_norm_weight}, {"self_attn.k_norm.weight", &b.k_norm_weight},
        {"mlp.gate_proj.weight", &b.gate_proj_weight}, {"mlp.up_proj.weight", &b.up_proj_weight}, {"mlp.down_proj.weight", &b.down_proj_weight}};
    auto it = slots.find(m[2].str());
    if (it == slots.end()) throw std::runtime_error("Unknown Gemma block weight: " + m[2].str());
    *it->second = t;
}

void GemmaModel::init_lora_modules() {
    for (auto& b : blocks_) {
        if (b.lora_initialized) continue;
        b.q_proj_lora = std::make_unique<LoRALinear>(b.q_proj_weight);
        b.k_proj_lora = std::make_unique<LoRALinear>(b.k_proj_weight);
        b.v_proj_lora = std::make_unique<LoRALinear>(b.v_proj_weight);
        b.o_proj_lora = std::make_unique<LoRALinear>(b.o_proj_weight);
        b.gate_proj_lora = std::make_unique<LoRALinear>(b.gate_proj_weight);
        b.up_proj_lora = std::make_unique<LoRALinear>(b.up_proj_weight);
        b.down_proj_lora = std::make_unique<LoRALinear>(b.down_proj_weight);
        b.lora_initialized = true;
    }
}

GemmaBlockWeights& GemmaModel::get_block(int i) {
    if (i < 0 || i >= (int)blocks_.size()) throw std::out_of_range("Gemma block index");
    return blocks_[(size_t)i];
}
const GemmaBlockWeights& GemmaModel::get_block(int i) const {
    if (i < 0 || i >= (int)blocks_.size()) throw std::out_of_range("Gemma block index");
    return blocks_[(size_t)i];
}

std::vector<TensorPtr> GemmaModel::parameters() const {
    std::vector<TensorPtr> p = {embed_weight_, norm_weight_, lm_head_weight_};
    for (const auto& b : blocks_)
        for (const TensorPtr& t : {b.input_layernorm_weight, b.post_attention_layernorm_weight, b.pre_feedforward_layernorm_weight,
                                   b.post_feedforward_layernorm_weight, b.q_proj_weight, b.k_proj_weight, b.v_proj_weight, b.o_proj_weight,
                                   b.q_norm_weight, b.k_norm_weight, b.gate_proj_weight, b.up_proj_weight, b.down_proj_weight})
            p.push_back(t);
    return p;
}

std::vector<TensorPtr> GemmaModel::get_lora_parameters() const { return impl_->lora_parameters(); }

static void each_module(GemmaBlockWeights& b, void (LoRALinear::*fn)()) {
    for (LoRALinear* m : {b.q_proj_lora.get(), b.k_proj_lora.get(), b.v_proj_lora.get(), b.o_proj_lora.get(), b.gate_proj_lora.get(),
                          b.up_proj_lora.get(), b.down_proj_lora.get()})
        if (m) (m->*fn)();
}
void GemmaModel::merge_lora() {
    for (auto& b : blocks_)
        if (b.lora_initialized) each_module(b, &LoRALinear::merge_to_base);
}
void GemmaModel::unmerge_lora() {
    for (auto& b : blocks_)
        if (b.lora_initialized) each_module(b, &LoRALinear::unmerge_from_base);
}

void GemmaModel::request_embedding_dump(int step, const std::string& dir) {
    dump_request_.active = true; dump_request_.target_step = step; dump_request_.output_dir = dir; dump_request_.fulfilled = false;
}
void GemmaModel::enable_debug_dump(const std::string& dir, const std::vector<int>& layers) {
    debug_.enabled = true; debug_.dir = dir; debug_.layers.clear(); debug_.tensors.clear();
    for (int l : layers) debug_.layers.insert(l);
    std::cerr << "[GemmaModel] per-layer tensor dumps are not produced by the fused device path" << std::endl;
}
void GemmaModel::disable_debug_dump() { debug_ = DebugConfig{}; }
void GemmaModel::set_numeric_perturb(bool enable, const std::string&, int64_t, float) {
    if (enable) throw std::runtime_error("GemmaModel::set_numeric_perturb: intermediate tensors are not addressable on the fused device path");
}
void GemmaModel::dump_layer_norm_weights(int, const std::string&) const {}

}  // namespace ops
