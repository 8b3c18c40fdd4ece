#include "qwen_model.h"

#include <cmath>
#include <cstring>
#include <iostream>
#include <random>
#include <regex>
#include <stdexcept>

#include "../core/ops.h"
#include "engine_model.h"
#include "json_fields.h"

namespace ops {

QwenConfig QwenConfig::from_pretrained(const std::string& path) {
    const std::string js = detail::read_config_text(path);
    QwenConfig c;
    c.vocab_size = detail::json_int(js, "vocab_size", c.vocab_size);
    c.hidden_size = detail::json_int(js, "hidden_size", c.hidden_size);
    c.intermediate_size = detail::json_int(js, "intermediate_size", c.intermediate_size);
    c.num_hidden_layers = detail::json_int(js, "num_hidden_layers", c.num_hidden_layers);
    c.num_attention_heads = detail::json_int(js, "num_attention_heads", c.num_attention_heads);
    c.num_key_value_heads = detail::json_int(js, "num_key_value_heads", c.num_key_value_heads);
    c.max_position_embeddings = detail::json_int(js, "max_position_embeddings", c.max_position_embeddings);
    c.bos_token_id = detail::json_int(js, "bos_token_id", c.bos_token_id);
    c.eos_token_id = detail::json_int(js, "eos_token_id", c.eos_token_id);
    c.pad_token_id = detail::json_int(js, "pad_token_id", c.pad_token_id);
    c.rms_norm_eps = detail::json_float(js, "rms_norm_eps", c.rms_norm_eps);
    c.rope_theta = detail::json_float(js, "rope_theta", c.rope_theta);
    c.hidden_act = detail::json_string(js, "hidden_act", c.hidden_act);
    return c;
}

static TensorPtr zeros_f32(std::vector<int64_t> shape) { return std::make_shared<Tensor>(shape, kFloat32, kCPU); }

QwenModel::QwenModel(const QwenConfig& cfg) : config_(cfg) {
    const int64_t H = cfg.hidden_size, I = cfg.intermediate_size;
    if (cfg.num_attention_heads <= 0 || H % cfg.num_attention_heads != 0) throw std::runtime_error("QwenModel: hidden_size must be divisible by the head count");
    const int64_t hd = H / cfg.num_attention_heads, KD = cfg.num_key_value_heads * hd;
    embed_tokens_ = zeros_f32({cfg.vocab_size, H});
    final_norm_weight_ = zeros_f32({H});
    layers_.resize((size_t)cfg.num_hidden_layers);
    for (auto& b : layers_) {
        b.input_norm_weight = zeros_f32({H}); b.post_norm_weight = zeros_f32({H});
        b.q_proj_weight = zeros_f32({H, H}); b.q_proj_bias = zeros_f32({H});
        b.k_proj_weight = zeros_f32({H, KD}); b.k_proj_bias = zeros_f32({KD});
        b.v_proj_weight = zeros_f32({H, KD}); b.v_proj_bias = zeros_f32({KD});
        b.o_proj_weight = zeros_f32({H, H});
        b.gate_proj_weight = zeros_f32({H, I}); b.up_proj_weight = zeros_f32({H, I}); b.down_proj_weight = zeros_f32({I, H});
    }
    mft_model_config_t a{};
    a.family = MFT_FAMILY_QWEN;
    a.vocab = cfg.vocab_size; a.hidden = cfg.hidden_size; a.inter = cfg.intermediate_size; a.layers = cfg.num_hidden_layers;
    a.n_heads = cfg.num_attention_heads; a.n_kv_heads = cfg.num_key_value_heads; a.head_dim = (int)hd;
    a.norm_eps = cfg.rms_norm_eps; a.rope_theta = cfg.rope_theta; a.attn_scale = 1.0f / std::sqrt((float)hd);
    a.gpt2_detach_attn = 1;
    impl_ = std::make_shared<detail::EngineModel>(
        a, [this] { return parameters(); },
        [this](int layer, uint32_t target) -> LoRALinear* {
            QwenBlock& b = layers_[(size_t)layer];
            switch (target) {
                case MFT_LORA_Q: return b.q_lin.get();
                case MFT_LORA_K: return b.k_lin.get();
                case MFT_LORA_V: return b.v_lin.get();
                case MFT_LORA_O: return b.o_lin.get();
                default: return nullptr;
            }
        });
}

QwenModel::~QwenModel() = default;

TensorPtr QwenModel::forward_hidden(const TensorPtr& ids, const TensorPtr& mask) { return impl_->forward_hidden(ids, mask); }
TensorPtr QwenModel::forward(const TensorPtr& ids, const TensorPtr& mask) { return impl_->forward(ids, mask); }
TensorPtr QwenModel::lm_head(const TensorPtr& hidden) {
    if (auto lazy = impl_->lm_head_of(hidden)) return lazy;
    return matmul_rhs_T(hidden, embed_tokens_);
}

void QwenModel::assign_weight(const std::string& key, const TensorPtr& t) {
    if (key == "embed_tokens.weight") { embed_tokens_ = t; return; }
    if (key == "final_norm.weight") { final_norm_weight_ = t; return; }
    std::smatch m;
    if (!std::regex_match(key, m, std::regex(R"(layers\.(\d+)\.(.+))"))) return;
    const int idx = std::stoi(m[1].str());
    if (idx < 0 || idx >= config_.num_hidden_layers) throw std::runtime_error("bad layer idx");
    QwenBlock& b = layers_[(size_t)idx];
    const std::unordered_map<std::string, TensorPtr*> slots = {
        {"input_norm.weight", &b.input_norm_weight}, {"post_norm.weight", &b.post_norm_weight},
        {"self_attn.q_proj.weight", &b.q_proj_weight}, {"self_attn.q_proj.bias", &b.q_proj_bias},
        {"self_attn.k_proj.weight", &b.k_proj_weight}, {"self_attn.k_proj.bias", &b.k_proj_bias},
        {"self_attn.v_proj.weight", &b.v_proj_weight}, {"self_attn.v_proj.bias", &b.v_proj_bias},
        {"self_attn.o_proj.weight", &b.o_proj_weight}, {"mlp.gate_proj.weight", &b.gate_proj_weight},
        {"mlp.up_proj.weight", &b.up_proj_weight}, {"mlp.down_proj.weight", &b.down_proj_weight}};
    auto it = slots.find(m[2].str());
    if (it != slots.end()) *it->second = t;
}

void QwenModel::ensure_modules(QwenBlock& b) {
    b.q_lin = std::make_unique<LoRALinear>(b.q_proj_weight, b.q_proj_bias);
    b.k_lin = std::make_unique<LoRALinear>(b.k_proj_weight, b.k_proj_bias);
    b.v_lin = std::make_unique<LoRALinear>(b.v_proj_weight, b.v_proj_bias);
    b.o_lin = std::make_unique<LoRALinear>(b.o_proj_weight, nullptr);
}

void QwenModel::init_lora(int rank, float alpha, float /*dropout: never applied by the forward pass*/, bool qv_only, uint64_t seed) {
    if (rank <= 0) throw std::runtime_error("QwenModel::init_lora: rank must be positive");
    const float scale = alpha / (float)rank;
    std::mt19937 rng(static_cast<uint32_t>(seed));
    std::uniform_real_distribution<float> dist(-0.01f, 0.01f);
    const int64_t H = config_.hidden_size, KD = (int64_t)config_.num_key_value_heads * (H / config_.num_attention_heads);
    auto make = [&](int64_t in, int64_t out) {
        auto A = zeros_f32({in, rank});
        auto B = zeros_f32({rank, out});
        float* a = A->data<float>();
        for (int64_t i = 0; i < in * rank; ++i) a[i] = dist(rng);
        A->set_requires_grad(true);
        B->set_requires_grad(true);
        return std::make_pair(A, B);
    };
    for (auto& b : layers_) {
        ensure_modules(b);
        auto q = make(H, H);
        auto v = make(H, KD);
        b.q_lin->attach_lora(q.first, q.second, scale);
        b.v_lin->attach_lora(v.first, v.second, scale);
        if (!qv_only) {
            auto k = make(H, KD);
            auto o = make(H, H);
            b.k_lin->attach_lora(k.first, k.second, scale);
            b.o_lin->attach_lora(o.first, o.second, scale);
        }
        b.lora_initialized = true;
    }
}

std::vector<TensorPtr> QwenModel::get_lora_parameters() const { return impl_->lora_parameters(); }

std::vector<TensorPtr> QwenModel::parameters() const {
    std::vector<TensorPtr> p = {embed_tokens_, final_norm_weight_};
    for (const auto& b : layers_)
        for (const TensorPtr& t : {b.input_norm_weight, b.post_norm_weight, b.q_proj_weight, b.q_proj_bias, b.k_proj_weight, b.k_proj_bias,
                                   b.v_proj_weight, b.v_proj_bias, b.o_proj_weight, b.gate_proj_weight, b.up_proj_weight, b.down_proj_weight})
            p.push_back(t);
    return p;
}

void QwenModel::freeze_base() {
    for (auto& t : parameters())
        if (t) t->set_requires_grad(false);
}

}  // namespace ops
