#include "auto_model.h"

#include <algorithm>
#include <stdexcept>

#include "../core/memory_manager.h"

namespace ops {

namespace {
bool has(const std::vector<std::string>& v, const std::string& s) { return std::find(v.begin(), v.end(), s) != v.end(); }
bool any_of_names(const std::vector<std::string>& v, std::initializer_list<const char*> names) {
    for (const char* n : names)
        if (has(v, n)) return true;
    return false;
}
}  // namespace

std::unique_ptr<AutoModelForCausalLM> AutoModelForCausalLM::from_pretrained(const std::string& dir, const AutoModelLoadOptions& options) {
    std::unique_ptr<AutoModelForCausalLM> m(new AutoModelForCausalLM(dir, ModelRegistry::inspect_pretrained(dir)));
    switch (m->spec_.family) {
        case ModelFamily::GPT2: {
            const GPT2Config cfg = GPT2Config::from_pretrained(dir);
            m->gpt2_ = std::make_unique<GPT2Model>(cfg);
            if (cfg.tie_word_embeddings) m->gpt2_->tie_weights();
            break;
        }
        case ModelFamily::Gemma: m->gemma_ = std::make_unique<GemmaModel>(GemmaTextConfig::from_pretrained(dir)); break;
        case ModelFamily::Qwen: m->qwen_ = std::make_unique<QwenModel>(QwenConfig::from_pretrained(dir + "/config.json")); break;
        default: throw std::runtime_error("AutoModelForCausalLM: unsupported model family");
    }
    if (options.load_weights) m->load_pretrained_weights(options);
    return m;
}

void AutoModelForCausalLM::load_pretrained_weights(const AutoModelLoadOptions& options) {
    SafeTensorsModelReader reader(model_dir_);
    reader.parse_headers();
    SafeTensorsLoadOptions lo = options.safetensors_options;
    lo.verbose = options.verbose;
    // GPT-2 checkpoints store linears as [in, out] already; HuggingFace Gemma / Qwen linears are [out, in]
    lo.transpose_linear = spec_.family != ModelFamily::GPT2;
    if (gpt2_) {
        for (const auto& kv : reader.load_tensors_mapped(GPT2KeyMapper::generate_gpt2_mapping(gpt2_->config().n_layer), lo)) gpt2_->assign_weight(kv.first, kv.second);
    } else if (gemma_) {
        for (const auto& kv : reader.load_tensors_mapped(GemmaKeyMapper::generate_gemma_mapping(gemma_->config().num_hidden_layers), lo)) gemma_->assign_weight(kv.first, kv.second);
    } else if (qwen_) {
        for (const auto& kv : reader.load_tensors_mapped(QwenKeyMapper::generate_qwen_mapping(qwen_->config().num_hidden_layers), lo)) qwen_->assign_weight(kv.first, kv.second);
        MemoryManager::instance().clear_unused_memory();
    }
}

TensorPtr AutoModelForCausalLM::forward(const TensorPtr& ids, const TensorPtr& mask) {
    if (gpt2_) return gpt2_->forward(ids, mask);
    if (gemma_) return gemma_->forward(ids, mask);
    if (qwen_) return qwen_->forward(ids, mask);
    throw std::runtime_error("AutoModelForCausalLM: unsupported model family");
}

void AutoModelForCausalLM::init_lora(const AutoLoraConfig& c) {
    const auto& t = c.target_modules;
    if (gpt2_) {
        LoraSpec s;
        s.rank = c.rank; s.alpha = c.alpha; s.dropout = c.dropout;
        s.split_qkv = !any_of_names(t, {"c_attn", "attn_qkv"});
        if (!t.empty()) {
            s.targets.clear();
            if (any_of_names(t, {"attn_qkv", "c_attn", "q_proj", "k_proj", "v_proj"})) s.targets.push_back(LoraTarget::AttnQKV);
            if (any_of_names(t, {"attn_proj", "c_proj", "o_proj"})) s.targets.push_back(LoraTarget::AttnProj);
            if (any_of_names(t, {"mlp_fc_in", "c_fc"})) s.targets.push_back(LoraTarget::MlpFcIn);
            if (any_of_names(t, {"mlp_fc_out", "mlp_c_proj"})) s.targets.push_back(LoraTarget::MlpFcOut);
            if (s.targets.empty()) throw std::runtime_error("AutoModelForCausalLM: no supported GPT-2 LoRA targets requested");
        }
        for (int i = 0; i < gpt2_->config().n_layer; ++i) {          // a second init_lora replaces the adapters
            GPT2BlockWeights& b = gpt2_->get_block(i);
            for (LoRALinear* m : {b.qkv_lin.get(), b.proj_lin.get(), b.fc_in_lin.get(), b.fc_out_lin.get()})
                if (m) m->clear_lora();
        }
        gpt2_->init_lora_modules();
        gpt2_lora_ = std::make_unique<LoraInjector>();
        gpt2_lora_->inject(*gpt2_, s);
    } else if (gemma_) {
        GemmaLoraSpec s;
        s.rank = c.rank; s.alpha = c.alpha; s.dropout = c.dropout;
        if (!t.empty()) s.target_modules = t;
        if (gemma_lora_)
            for (int i = 0; i < gemma_->config().num_hidden_layers; ++i) {
                GemmaBlockWeights& b = gemma_->get_block(i);
                for (LoRALinear* m : {b.q_proj_lora.get(), b.k_proj_lora.get(), b.v_proj_lora.get(), b.o_proj_lora.get(), b.gate_proj_lora.get(),
                                      b.up_proj_lora.get(), b.down_proj_lora.get()})
                    if (m) m->clear_lora();
            }
        gemma_lora_ = std::make_unique<GemmaLoraInjector>();
        gemma_lora_->inject(*gemma_, s);
    } else if (qwen_) {
        const bool qv_only = !t.empty() && has(t, "q_proj") && has(t, "v_proj") && !has(t, "k_proj") && !has(t, "o_proj");
        qwen_->init_lora(c.rank, c.alpha, c.dropout, qv_only, c.seed);
        qwen_->freeze_base();
    } else {
        throw std::runtime_error("AutoModelForCausalLM: unsupported model family");
    }
}

std::vector<TensorPtr> AutoModelForCausalLM::parameters() {
    if (gpt2_) return gpt2_->parameters();
    if (gemma_) return gemma_->parameters();
    if (qwen_) return qwen_->parameters();
    throw std::runtime_error("AutoModelForCausalLM: unsupported model family");
}

std::vector<TensorPtr> AutoModelForCausalLM::trainable_parameters() {
    if (gpt2_) return gpt2_->get_lora_parameters();
    if (gemma_) return gemma_->get_lora_parameters();
    if (qwen_) return qwen_->get_lora_parameters();
    throw std::runtime_error("AutoModelForCausalLM: unsupported model family");
}

}  // namespace ops
