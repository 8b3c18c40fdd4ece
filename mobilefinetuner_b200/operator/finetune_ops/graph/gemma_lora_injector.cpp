#include "gemma_lora_injector.h"

#include <algorithm>
#include <cctype>
#include <cmath>
#include <iostream>
#include <map>
#include <random>
#include <sstream>
#include <stdexcept>

#include "../core/ops.h"
#include "lora_file.h"
#include "lora_saver.h"

namespace ops {

namespace {
struct Linear { LoRALinear* module; TensorPtr weight; };
Linear find_linear(GemmaBlockWeights& b, const std::string& name) {
    if (name == "q_proj") return {b.q_proj_lora.get(), b.q_proj_weight};
    if (name == "k_proj") return {b.k_proj_lora.get(), b.k_proj_weight};
    if (name == "v_proj") return {b.v_proj_lora.get(), b.v_proj_weight};
    if (name == "o_proj") return {b.o_proj_lora.get(), b.o_proj_weight};
    if (name == "gate_proj") return {b.gate_proj_lora.get(), b.gate_proj_weight};
    if (name == "up_proj") return {b.up_proj_lora.get(), b.up_proj_weight};
    if (name == "down_proj") return {b.down_proj_lora.get(), b.down_proj_weight};
    return {nullptr, nullptr};
}
const std::pair<const char*, const char*> kFileNames[] = {{"attn.q", "q_proj"}, {"attn.k", "k_proj"}, {"attn.v", "v_proj"}, {"attn.proj", "o_proj"},
                                                          {"mlp.gate", "gate_proj"}, {"mlp.up", "up_proj"}, {"mlp.down", "down_proj"}};
void clear_all(GemmaBlockWeights& b) {
    for (const auto& n : kFileNames)
        if (LoRALinear* m = find_linear(b, n.second).module) m->clear_lora();
}
// A ~ U(+-1/sqrt(in)) [rank, in] (what PEFT's kaiming_uniform_(a = sqrt(5)) amounts to), B = 0 [out, rank].  One
// generator, seeded with 42, serves every pair of the process, in creation order.
std::pair<TensorPtr, TensorPtr> new_pair(int64_t in, int64_t out, int rank) {
    static std::mt19937 rng(42);
    const float bound = 1.0f / std::sqrt((float)in);
    std::uniform_real_distribution<float> dist(-bound, bound);
    auto A = zeros({rank, in}, kFloat32, kCPU);
    float* a = A->data<float>();
    for (int64_t i = 0; i < A->numel(); ++i) a[i] = dist(rng);
    auto B = zeros({out, rank}, kFloat32, kCPU);
    A->set_requires_grad(true);
    B->set_requires_grad(true);
    return {A, B};
}
std::string num(float v) { std::ostringstream os; os << v; return os.str(); }
}  // namespace

void GemmaLoraInjector::inject(GemmaModel& model, const GemmaLoraSpec& spec) {
    if (spec.rank <= 0) throw std::runtime_error("GemmaLoraInjector::inject: rank must be positive");
    model_ = &model;
    spec_ = spec;
    num_layers_ = model.config().num_hidden_layers;
    model.init_lora_modules();
    attached_modules_ = 0;
    std::vector<int> layers = spec.layers;
    if (layers.empty())
        for (int i = 0; i < num_layers_; ++i) layers.push_back(i);
    const float scale = spec.alpha / (float)spec.rank;
    for (int l : layers) {
        GemmaBlockWeights& b = model.get_block(l);
        for (const std::string& name : spec.target_modules) {
            Linear lin = find_linear(b, name);
            if (!lin.module || !lin.weight || lin.weight->shape().size() != 2) {
                std::cerr << "[GemmaLoraInjector] Skip module " << name << " in layer " << l << std::endl;
                continue;
            }
            const int64_t in = lin.weight->shape()[0], out = lin.weight->shape()[1];      // weights are [in, out]
            auto ab = new_pair(in, out, spec.rank);
            lin.module->attach_lora(ab.first, ab.second, scale, 0, (int)out);
            ++attached_modules_;
        }
    }
    std::cout << "[GemmaLoraInjector] " << attached_modules_ << " adapters on " << layers.size() << " layers (rank " << spec.rank << ", alpha "
              << spec.alpha << ")" << std::endl;
}

std::vector<TensorPtr> GemmaLoraInjector::get_trainable_params() const {
    if (!model_) return {};
    auto params = model_->get_lora_parameters();
    for (auto& p : params) p->set_requires_grad(true);
    return params;
}

void GemmaLoraInjector::print_info() const {
    std::cout << "[GemmaLoraInjector] rank " << spec_.rank << ", alpha " << spec_.alpha << ", dropout " << spec_.dropout << ", adapters "
              << attached_modules_ << ", targets";
    for (const auto& t : spec_.target_modules) std::cout << " " << t;
    std::cout << std::endl;
}

void GemmaLoraInjector::save_lora_safetensors(const std::string& path) const {
    if (!model_) { std::cerr << "[GemmaLoraInjector] save_lora_safetensors: model not set" << std::endl; return; }
    std::map<std::string, TensorPtr> state;
    std::vector<std::string> targets;
    for (int i = 0; i < model_->config().num_hidden_layers; ++i) {
        GemmaBlockWeights& b = const_cast<GemmaModel*>(model_)->get_block(i);
        for (const auto& n : kFileNames) {
            LoRALinear* m = find_linear(b, n.second).module;
            if (!m || m->slices().empty()) continue;
            if (std::find(targets.begin(), targets.end(), n.first) == targets.end()) targets.push_back(n.first);
            const auto& sl = m->slices();
            for (size_t k = 0; k < sl.size(); ++k) {
                std::string base = "layer." + std::to_string(i) + "." + n.first;
                if (sl.size() > 1) base += "." + std::to_string(k);
                state[base + ".lora_A"] = sl[k].A;
                state[base + ".lora_B"] = sl[k].B;
            }
        }
    }
    std::sort(targets.begin(), targets.end());
    std::string csv;
    for (size_t i = 0; i < targets.size(); ++i) csv += (i ? "," : "") + targets[i];
    detail::write_adapter_file(path, state, {{"rank", std::to_string(spec_.rank)}, {"alpha", num(spec_.alpha)}, {"dropout", num(spec_.dropout)}, {"targets", csv}});
    std::cout << "[GemmaLoraInjector] Saved " << state.size() << " LoRA tensors to " << path << std::endl;
}

void GemmaLoraInjector::load_lora_safetensors(const std::string& path) {
    if (!model_) throw std::logic_error("GemmaLoraInjector::load_lora_safetensors requires an attached GemmaModel");
    model_->init_lora_modules();
    num_layers_ = model_->config().num_hidden_layers;
    const LoRAState st = LoraSaver::load_safetensors(path);
    struct Pair { int layer = -1; std::string target; TensorPtr A, B; };
    std::map<std::string, Pair> groups;
    for (const auto& kv : st.tensors) {
        int layer = -1;
        std::string target, ab;
        if (!LoraSaver::parse_peft_key(kv.first, layer, target, ab)) continue;
        if (layer < 0 || layer >= num_layers_) throw std::runtime_error("GemmaLoraInjector::load_lora_safetensors layer out of range: " + std::to_string(layer));
        Pair& p = groups[std::to_string(layer) + ":" + target];
        p.layer = layer;
        p.target = target;
        (ab == "A" ? p.A : p.B) = kv.second;
    }
    for (int l = 0; l < num_layers_; ++l) clear_all(model_->get_block(l));
    const float scale = st.alpha / (st.rank > 0 ? (float)st.rank : 1.0f);
    attached_modules_ = 0;
    std::vector<std::string> modules;
    for (auto& kv : groups) {
        Pair& p = kv.second;
        if (!p.A || !p.B) throw std::runtime_error("GemmaLoraInjector::load_lora_safetensors missing A/B pair for " + kv.first);
        std::string target = p.target;                                   // "attn.q.1" (several slices on one linear) -> "attn.q"
        const size_t dot = target.rfind('.');
        if (dot != std::string::npos && dot + 1 < target.size() && std::all_of(target.begin() + (long)dot + 1, target.end(), [](unsigned char c) { return std::isdigit(c); }))
            target.erase(dot);
        std::string module;
        for (const auto& n : kFileNames)
            if (target == n.first) module = n.second;
        if (module.empty()) throw std::runtime_error("GemmaLoraInjector::load_lora_safetensors unsupported target: " + p.target);
        Linear lin = find_linear(model_->get_block(p.layer), module);
        if (!lin.module || !lin.weight) throw std::runtime_error("GemmaLoraInjector::load_lora_safetensors unresolved module: " + module);
        p.A->set_requires_grad(true);
        p.B->set_requires_grad(true);
        lin.module->attach_lora(p.A, p.B, scale, 0, (int)lin.weight->shape()[1]);
        ++attached_modules_;
        if (std::find(modules.begin(), modules.end(), module) == modules.end()) modules.push_back(module);
    }
    spec_.rank = st.rank;
    spec_.alpha = st.alpha;
    spec_.dropout = st.dropout;
    if (!modules.empty()) spec_.target_modules = modules;
    std::cout << "[GemmaLoraInjector] Loaded " << attached_modules_ << " adapters from " << path << std::endl;
}

void GemmaLoraInjector::merge_all(GemmaModel& model) { model.merge_lora(); }
void GemmaLoraInjector::unmerge_all(GemmaModel& model) { model.unmerge_lora(); }

}  // namespace ops
