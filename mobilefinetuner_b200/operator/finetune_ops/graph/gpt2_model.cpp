#include "gpt2_model.h"

#include <cmath>
#include <iostream>
#include <regex>
#include <stdexcept>

#include "engine_model.h"
#include "json_fields.h"

namespace ops {

GPT2Config GPT2Config::from_pretrained(const std::string& path) {
    const std::string js = detail::read_config_text(path);
    GPT2Config c;
    c.vocab_size = detail::json_int(js, "vocab_size", c.vocab_size);
    c.n_positions = detail::json_int(js, "n_positions", detail::json_int(js, "n_ctx", c.n_positions));
    c.n_embd = detail::json_int(js, "n_embd", c.n_embd);
    c.n_layer = detail::json_int(js, "n_layer", c.n_layer);
    c.n_head = detail::json_int(js, "n_head", c.n_head);
    c.layernorm_eps = detail::json_float(js, "layer_norm_epsilon", c.layernorm_eps);
    c.tie_word_embeddings = true;
    c.use_cache = false;
    return c;
}

static TensorPtr zeros_f32(std::vector<int64_t> shape) { return std::make_shared<Tensor>(shape, kFloat32, kCPU); }

GPT2Model::GPT2Model(const GPT2Config& config) : config_(config) {
    const int64_t C = config_.n_embd;
    if (config_.n_head <= 0 || C % config_.n_head != 0) throw std::runtime_error("GPT2Model: n_embd must be divisible by n_head");
    wte_weight_ = zeros_f32({config_.vocab_size, C});
    wpe_weight_ = zeros_f32({config_.n_positions, C});
    blocks_.resize((size_t)config_.n_layer);
    for (auto& b : blocks_) {
        b.ln_1_weight = zeros_f32({C}); b.ln_1_bias = zeros_f32({C});
        b.attn_qkv_weight = zeros_f32({C, 3 * C}); b.attn_qkv_bias = zeros_f32({3 * C});
        b.attn_proj_weight = zeros_f32({C, C}); b.attn_proj_bias = zeros_f32({C});
        b.ln_2_weight = zeros_f32({C}); b.ln_2_bias = zeros_f32({C});
        b.mlp_fc_in_weight = zeros_f32({C, 4 * C}); b.mlp_fc_in_bias = zeros_f32({4 * C});
        b.mlp_fc_out_weight = zeros_f32({4 * C, C}); b.mlp_fc_out_bias = zeros_f32({C});
    }
    ln_f_weight_ = zeros_f32({C});
    ln_f_bias_ = zeros_f32({C});

    mft_model_config_t a{};
    a.family = MFT_FAMILY_GPT2;
    a.vocab = config_.vocab_size; a.hidden = config_.n_embd; a.inter = 4 * config_.n_embd; a.layers = config_.n_layer;
    a.n_heads = a.n_kv_heads = config_.n_head; a.head_dim = config_.n_embd / config_.n_head;
    a.n_positions = config_.n_positions; a.norm_eps = config_.layernorm_eps;
    a.attn_scale = 1.0f / std::sqrt((float)a.head_dim);
    a.gpt2_detach_attn = 1;         // the reference's Q/K/V split severs autograd (gpt2_model.cpp:560-581): reproduced
    impl_ = std::make_shared<detail::EngineModel>(
        a, [this] { return parameters(); },
        [this](int layer, uint32_t target) -> LoRALinear* {
            GPT2BlockWeights& b = blocks_[(size_t)layer];
            switch (target) {
                case MFT_LORA_Q: return b.qkv_lin.get();
                case MFT_LORA_O: return b.proj_lin.get();
                case MFT_LORA_GATE: return b.fc_in_lin.get();
                case MFT_LORA_DOWN: return b.fc_out_lin.get();
                default: return nullptr;
            }
        });
}

GPT2Model::~GPT2Model() = default;

TensorPtr GPT2Model::forward(const TensorPtr& input_ids, const TensorPtr& attention_mask) {
    if (input_ids && input_ids->shape().size() == 2 && input_ids->shape()[1] > config_.n_positions)
        throw std::runtime_error("GPT2Model::forward: sequence longer than n_positions");
    return impl_->forward(input_ids, attention_mask);
}

void GPT2Model::tie_weights() { weights_tied_ = true; }        // the lm head always reads wte

void GPT2Model::assign_weight(const std::string& key, const TensorPtr& t) {
    if (key == "wte.weight") { wte_weight_ = t; return; }
    if (key == "wpe.weight") { wpe_weight_ = t; return; }
    if (key == "ln_f.weight") { ln_f_weight_ = t; return; }
    if (key == "ln_f.bias") { ln_f_bias_ = t; return; }
    std::smatch m;
    if (!std::regex_match(key, m, std::regex(R"(blocks\.(\d+)\.(.+))"))) {
        std::cerr << "[GPT2Model] unknown weight key " << key << std::endl;
        return;
    }
    const int idx = std::stoi(m[1].str());
    if (idx < 0 || idx >= config_.n_layer) throw std::runtime_error("Invalid block index: " + std::to_string(idx));
    GPT2BlockWeights& b = blocks_[(size_t)idx];
    const std::string leaf = m[2].str();
    const std::unordered_map<std::string, TensorPtr*> slots = {
        {"ln_1.weight", &b.ln_1_weight}, {"ln_1.bias", &b.ln_1_bias}, {"attn.qkv.weight", &b.attn_qkv_weight}, {"attn.qkv.bias", &b.attn_qkv_bias},
        {"attn.proj.weight", &b.attn_proj_weight}, {"attn.proj.bias", &b.attn_proj_bias}, {"ln_2.weight", &b.ln_2_weight}, {"ln_2.bias", &b.ln_2_bias},
        {"mlp.fc_in.weight", &b.mlp_fc_in_weight}, {"mlp.fc_in.bias", &b.mlp_fc_in_bias}, {"mlp.fc_out.weight", &b.mlp_fc_out_weight},
        {"mlp.fc_out.bias", &b.mlp_fc_out_bias}};
    auto it = slots.find(leaf);
    if (it == slots.end()) { std::cerr << "[GPT2Model] unknown weight key " << key << std::endl; return; }
    *it->second = t;
}

std::vector<TensorPtr> GPT2Model::parameters() {
    std::vector<TensorPtr> p = {wte_weight_, wpe_weight_};
    for (auto& b : blocks_)
        for (const TensorPtr& t : {b.ln_1_weight, b.ln_1_bias, b.attn_qkv_weight, b.attn_qkv_bias, b.attn_proj_weight, b.attn_proj_bias,
                                   b.ln_2_weight, b.ln_2_bias, b.mlp_fc_in_weight, b.mlp_fc_in_bias, b.mlp_fc_out_weight, b.mlp_fc_out_bias})
            p.push_back(t);
    p.push_back(ln_f_weight_);
    p.push_back(ln_f_bias_);
    return p;
}

std::vector<TensorPtr> GPT2Model::trainable_parameters() {
    std::vector<TensorPtr> out;
    for (auto& t : get_lora_parameters())
        if (t && t->requires_grad()) out.push_back(t);
    return out;
}

void GPT2Model::freeze_base_parameters() {
    for (auto& t : parameters())
        if (t) t->set_requires_grad(false);
}

void GPT2Model::print_model_info() const {
    std::cout << "GPT-2: " << config_.n_layer << " layers, width " << config_.n_embd << ", " << config_.n_head << " heads, vocabulary "
              << config_.vocab_size << ", positions " << config_.n_positions << (weights_tied_ ? ", tied lm head" : "") << std::endl;
}

GPT2BlockWeights& GPT2Model::block_at(int i, const char* who) {
    if (i < 0 || i >= config_.n_layer) throw std::out_of_range(std::string(who) + ": layer index");
    return blocks_[(size_t)i];
}
std::pair<TensorPtr*, TensorPtr*> GPT2Model::attn_qkv_params(int i) { auto& b = block_at(i, "attn_qkv_params"); return {&b.attn_qkv_weight, &b.attn_qkv_bias}; }
std::pair<TensorPtr*, TensorPtr*> GPT2Model::attn_proj_params(int i) { auto& b = block_at(i, "attn_proj_params"); return {&b.attn_proj_weight, &b.attn_proj_bias}; }
std::pair<TensorPtr*, TensorPtr*> GPT2Model::mlp_fc_in_params(int i) { auto& b = block_at(i, "mlp_fc_in_params"); return {&b.mlp_fc_in_weight, &b.mlp_fc_in_bias}; }
std::pair<TensorPtr*, TensorPtr*> GPT2Model::mlp_fc_out_params(int i) { auto& b = block_at(i, "mlp_fc_out_params"); return {&b.mlp_fc_out_weight, &b.mlp_fc_out_bias}; }

void GPT2Model::init_lora_modules() {
    for (auto& b : blocks_) {
        if (b.lora_initialized) continue;
        b.qkv_lin = std::make_unique<LoRALinear>(b.attn_qkv_weight, b.attn_qkv_bias);
        b.proj_lin = std::make_unique<LoRALinear>(b.attn_proj_weight, b.attn_proj_bias);
        b.fc_in_lin = std::make_unique<LoRALinear>(b.mlp_fc_in_weight, b.mlp_fc_in_bias);
        b.fc_out_lin = std::make_unique<LoRALinear>(b.mlp_fc_out_weight, b.mlp_fc_out_bias);
        b.lora_initialized = true;
    }
}

std::vector<TensorPtr> GPT2Model::get_lora_parameters() { return impl_->lora_parameters(); }

}  // namespace ops
