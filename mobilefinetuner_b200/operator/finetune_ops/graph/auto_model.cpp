#include "auto_model.h"

#include <cmath>
#include <fstream>
#include <random>
#include <regex>
#include <sstream>
#include <stdexcept>

#include "../core/ops.h"

namespace ops {

namespace {
std::string slurp(const std::string& path) {
    std::ifstream f(path);
    if (!f.is_open()) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
bool find_number(const std::string& js, const std::string& key, double* out) {
    std::smatch m;
    if (std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*(-?[0-9][0-9eE\\.+-]*)"))) { *out = std::stod(m[1]); return true; }
    return false;
}
int geti(const std::string& js, const std::string& key, int dflt) { double v; return find_number(js, key, &v) ? (int)v : dflt; }
float getf(const std::string& js, const std::string& key, float dflt) { double v; return find_number(js, key, &v) ? (float)v : dflt; }
std::string gets(const std::string& js, const std::string& key, const std::string& dflt) {
    std::smatch m;
    return std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*\"([^\"]+)\"")) ? std::string(m[1]) : dflt;
}
void check(int32_t s, const char* what) { if (s != MFT_OK) throw std::runtime_error(std::string(what) + ": " + mft_last_error()); }
bool has(const std::vector<std::string>& v, const std::string& s) { for (auto& x : v) if (x == s) return true; return false; }
}  // namespace

std::string to_string(ModelFamily f) {
    switch (f) { case ModelFamily::GPT2: return "gpt2"; case ModelFamily::Gemma: return "gemma"; case ModelFamily::Qwen: return "qwen"; default: return "unknown"; }
}

ModelFamily ModelRegistry::infer_family(const std::string& dir) { return inspect_pretrained(dir).family; }
ModelArchitectureSpec ModelRegistry::inspect_pretrained(const std::string& dir) {
    ModelArchitectureSpec s;
    s.assets.model_dir = dir;
    s.assets.config_json_path = dir + "/config.json";
    const std::string js = slurp(s.assets.config_json_path);
    s.model_type = gets(js, "model_type", "");
    if (s.model_type.find("gpt2") != std::string::npos) { s.family = ModelFamily::GPT2; s.default_lora_targets = {"c_attn", "c_proj"}; s.tie_word_embeddings = true; }
    else if (s.model_type.find("gemma") != std::string::npos) { s.family = ModelFamily::Gemma; s.default_lora_targets = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"}; s.tie_word_embeddings = true; }
    else if (s.model_type.find("qwen") != std::string::npos) { s.family = ModelFamily::Qwen; s.default_lora_targets = {"q_proj", "k_proj", "v_proj", "o_proj"}; s.tie_word_embeddings = true; }
    else throw std::runtime_error("ModelRegistry: unsupported model_type '" + s.model_type + "'");
    return s;
}

AutoModelForCausalLM::~AutoModelForCausalLM() { if (engine_) mft_model_destroy(engine_); }

std::unique_ptr<AutoModelForCausalLM> AutoModelForCausalLM::from_pretrained(const std::string& dir, const AutoModelLoadOptions& opt) {
    if (opt.load_weights) throw std::runtime_error("AutoModelForCausalLM: weight files are ingested by the host loader; construct with load_weights=false and fill parameters()");
    auto spec = ModelRegistry::inspect_pretrained(dir);
    std::unique_ptr<AutoModelForCausalLM> m(new AutoModelForCausalLM(dir, spec));
    const std::string js = slurp(spec.assets.config_json_path);
    mft_model_config_t& c = m->cfg_;
    c.lora_rank = 0;
    c.gpt2_detach_attn = 1;
    if (spec.family == ModelFamily::GPT2) {
        c.family = MFT_FAMILY_GPT2;
        c.vocab = geti(js, "vocab_size", 50257); c.hidden = geti(js, "n_embd", 768); c.layers = geti(js, "n_layer", 12);
        c.n_heads = c.n_kv_heads = geti(js, "n_head", 12); c.head_dim = c.hidden / c.n_heads; c.inter = 4 * c.hidden;
        c.n_positions = geti(js, "n_positions", geti(js, "n_ctx", 1024)); c.norm_eps = 1e-5f;
        c.attn_scale = 1.0f / std::sqrt((float)c.head_dim);
    } else if (spec.family == ModelFamily::Qwen) {
        c.family = MFT_FAMILY_QWEN;
        c.vocab = geti(js, "vocab_size", 151936); c.hidden = geti(js, "hidden_size", 896); c.inter = geti(js, "intermediate_size", 4864);
        c.layers = geti(js, "num_hidden_layers", 24); c.n_heads = geti(js, "num_attention_heads", 14); c.n_kv_heads = geti(js, "num_key_value_heads", 2);
        c.head_dim = c.hidden / c.n_heads; c.norm_eps = getf(js, "rms_norm_eps", 1e-6f); c.rope_theta = getf(js, "rope_theta", 1e6f);
        c.attn_scale = 1.0f / std::sqrt((float)c.head_dim);
    } else {
        c.family = MFT_FAMILY_GEMMA;
        c.vocab = geti(js, "vocab_size", 262144); c.hidden = geti(js, "hidden_size", 640); c.inter = geti(js, "intermediate_size", 2048);
        c.layers = geti(js, "num_hidden_layers", 18); c.n_heads = geti(js, "num_attention_heads", 4); c.n_kv_heads = geti(js, "num_key_value_heads", 1);
        c.head_dim = geti(js, "head_dim", 256); c.norm_eps = getf(js, "rms_norm_eps", 1e-6f); c.rope_theta = getf(js, "rope_theta", 1e6f);
        c.rope_local_theta = getf(js, "rope_local_base_freq", 1e4f); c.sliding_window = geti(js, "sliding_window", 512);
        c.attn_scale = std::pow(getf(js, "query_pre_attn_scalar", (float)c.head_dim), -0.5f);
        // layer_types: "full_attention" every k-th layer; absent = all sliding (as the reference)
        c.global_every = 0;
        std::smatch mm;
        if (std::regex_search(js, mm, std::regex("\"layer_types\"\\s*:\\s*\\[([^\\]]*)\\]"))) {
            const std::string arr = mm[1];
            int idx = 0, first_full = -1;
            const std::regex item("\"([a-z_]+)\"");
            for (std::sregex_iterator it(arr.begin(), arr.end(), item), end; it != end; ++it, ++idx)
                if ((*it)[1] == "full_attention" && first_full < 0) first_full = idx;
            if (first_full >= 0) c.global_every = first_full + 1;
        }
    }
    // host-visible parameter tensors in the reference's parameters() order: shapes come from a throw-away engine description
    c.max_batch = 1; c.max_seq = 8;
    return m;
}

void AutoModelForCausalLM::init_lora(const AutoLoraConfig& lc) {
    if (engine_) { mft_model_destroy(engine_); engine_ = nullptr; }
    std::vector<std::string> t = lc.target_modules.empty() ? spec_.default_lora_targets : lc.target_modules;
    uint32_t mask = 0;
    if (has(t, "q_proj") || has(t, "c_attn") || has(t, "attn_qkv")) mask |= MFT_LORA_Q;
    if (cfg_.family != MFT_FAMILY_GPT2) { if (has(t, "k_proj")) mask |= MFT_LORA_K; if (has(t, "v_proj")) mask |= MFT_LORA_V; }
    if (has(t, "o_proj") || has(t, "c_proj") || has(t, "attn_proj")) mask |= MFT_LORA_O;
    if (has(t, "gate_proj") || has(t, "c_fc") || has(t, "mlp_fc_in")) mask |= MFT_LORA_GATE;
    if (has(t, "up_proj")) mask |= MFT_LORA_UP;
    if (has(t, "down_proj") || has(t, "mlp_c_proj") || has(t, "mlp_fc_out")) mask |= MFT_LORA_DOWN;
    if (cfg_.family == MFT_FAMILY_QWEN) mask &= (MFT_LORA_Q | MFT_LORA_K | MFT_LORA_V | MFT_LORA_O);   // the Qwen graph has no LoRA slots in its MLP
    cfg_.lora_rank = lc.rank; cfg_.lora_alpha = lc.alpha; cfg_.lora_targets = mask;
    lora_.clear();
    lora_dirty_ = true;
}

void AutoModelForCausalLM::ensure_engine(int batch, int seq) {
    detail::ensure_runtime();
    const bool too_small = engine_ && ((int64_t)batch * seq > (int64_t)cfg_.max_batch * cfg_.max_seq || seq > cfg_.max_seq);
    if (engine_ && !too_small) return;
    if (engine_) { sync_lora_to_host(); mft_model_destroy(engine_); engine_ = nullptr; }
    cfg_.max_batch = std::max(batch, 1); cfg_.max_seq = std::max(seq, 8);
    check(mft_model_create(&cfg_, detail::stream(), &engine_), "mft_model_create");
    params_dirty_ = lora_dirty_ = true;
}

std::vector<TensorPtr> AutoModelForCausalLM::parameters() {
    if (params_.empty()) {
        ensure_engine(cfg_.max_batch, cfg_.max_seq);
        const int n = mft_model_param_count(engine_);
        for (int i = 0; i < n; ++i) {
            int64_t r = 0, c = 0;
            check(mft_model_param_shape(engine_, i, &r, &c), "param shape");
            params_.push_back(std::make_shared<Tensor>(r == 1 ? std::vector<int64_t>{c} : std::vector<int64_t>{r, c}, kFloat32, kCPU));
        }
    }
    params_dirty_ = true;     // the caller is about to fill them
    return params_;
}

std::vector<TensorPtr> AutoModelForCausalLM::trainable_parameters() {
    if (cfg_.lora_rank <= 0) return {};
    if (lora_.empty()) {
        ensure_engine(cfg_.max_batch, cfg_.max_seq);
        const int n = mft_model_lora_count(engine_);
        std::mt19937 rng(42);
        for (int i = 0; i < n; ++i) {
            int64_t r = 0, c = 0;
            check(mft_model_lora_shape(engine_, i, &r, &c), "lora shape");
            auto t = std::make_shared<Tensor>(std::vector<int64_t>{r, c}, kFloat32, kCPU);
            if (i % 2 == 0) {       // A: small uniform values, B: zeros (the reference's initialisation)
                std::uniform_real_distribution<float> d(-0.01f, 0.01f);
                float* p = t->data<float>();
                for (int64_t k = 0; k < t->numel(); ++k) p[k] = d(rng);
            }
            t->set_requires_grad(true);
            lora_.push_back(t);
        }
        lora_dirty_ = true;
    }
    sync_lora_to_host();
    lora_dirty_ = true;       // handed out mutable: re-upload before the next step
    return lora_;
}

void AutoModelForCausalLM::sync_lora_to_host() {
    if (!engine_ || !lora_host_stale_) return;
    for (size_t i = 0; i < lora_.size(); ++i) check(mft_model_get_lora_host(engine_, (int)i, lora_[i]->data<float>()), "get lora");
    lora_host_stale_ = false;
}

float AutoModelForCausalLM::forward_backward(const TensorPtr& ids, const TensorPtr& labels) {
    if (!ids || !labels || ids->dtype() != kInt32 || labels->dtype() != kInt32 || ids->shape().size() != 2) throw std::runtime_error("forward_backward: expects int32 [B,S] ids and labels");
    const int B = (int)ids->shape()[0], S = (int)ids->shape()[1];
    ensure_engine(B, S);
    if (params_dirty_) {
        if (params_.empty()) throw std::runtime_error("forward_backward: parameters() were never filled");
        for (size_t i = 0; i < params_.size(); ++i) check(mft_model_set_param_host(engine_, (int)i, static_cast<const Tensor&>(*params_[i]).data<float>()), "set param");
        params_dirty_ = false;
    }
    if (lora_dirty_ && !lora_.empty()) {
        for (size_t i = 0; i < lora_.size(); ++i) check(mft_model_set_lora_host(engine_, (int)i, static_cast<const Tensor&>(*lora_[i]).data<float>()), "set lora");
        lora_dirty_ = false;
    }
    float loss = 0.f;
    int32_t nv = 0;
    check(mft_model_forward_backward(engine_, static_cast<const Tensor&>(*ids).data<int32_t>(), static_cast<const Tensor&>(*labels).data<int32_t>(), B, S, 0, &loss, &nv), "forward_backward");
    return loss;
}

float AutoModelForCausalLM::forward_loss(const TensorPtr& ids, const TensorPtr& labels) {
    const int B = (int)ids->shape()[0], S = (int)ids->shape()[1];
    ensure_engine(B, S);
    if (params_dirty_ || (lora_dirty_ && !lora_.empty())) {
        for (size_t i = 0; i < params_.size() && params_dirty_; ++i) check(mft_model_set_param_host(engine_, (int)i, static_cast<const Tensor&>(*params_[i]).data<float>()), "set param");
        for (size_t i = 0; i < lora_.size() && lora_dirty_; ++i) check(mft_model_set_lora_host(engine_, (int)i, static_cast<const Tensor&>(*lora_[i]).data<float>()), "set lora");
        params_dirty_ = lora_dirty_ = false;
    }
    float loss = 0.f;
    check(mft_model_forward_loss(engine_, static_cast<const Tensor&>(*ids).data<int32_t>(), static_cast<const Tensor&>(*labels).data<int32_t>(), B, S, &loss), "forward_loss");
    return loss;
}

void AutoModelForCausalLM::optimizer_step(float lr, float b1, float b2, float eps, float wd, float max_norm, float clip_eps) {
    if (!engine_) throw std::runtime_error("optimizer_step before any forward_backward");
    check(mft_model_optimizer_step(engine_, lr, b1, b2, eps, wd, max_norm, clip_eps), "optimizer_step");
    lora_host_stale_ = true;
}

std::vector<TensorPtr> AutoModelForCausalLM::lora_gradients() {
    std::vector<TensorPtr> g;
    if (!engine_) return g;
    for (size_t i = 0; i < lora_.size(); ++i) {
        if (!mft_model_lora_has_grad(engine_, (int)i)) { g.push_back(nullptr); continue; }
        auto t = std::make_shared<Tensor>(lora_[i]->shape(), kFloat32, kCPU);
        check(mft_model_get_lora_grad_host(engine_, (int)i, t->data<float>()), "get lora grad");
        g.push_back(t);
    }
    return g;
}

}  // namespace ops
