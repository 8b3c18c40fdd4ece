#include "lora_injector.h"

#include <cmath>
#include <iostream>
#include <random>
#include <stdexcept>

#include "../core/ops.h"
#include "lora_saver.h"

namespace ops {

void LoraState::init(int64_t in_features, int64_t out_features, int rank, float alpha, float dropout) {
    scale = alpha / (float)rank;
    dropout_p = dropout;
    enabled = true;
    A = std::make_shared<Tensor>(std::vector<int64_t>{in_features, rank}, kFloat32, kCPU);
    std::mt19937 gen(std::random_device{}());
    std::normal_distribution<float> dist(0.0f, 1.0f / std::sqrt((float)rank));
    float* a = A->data<float>();
    for (int64_t i = 0; i < A->numel(); ++i) a[i] = dist(gen);
    B = zeros({rank, out_features}, kFloat32, kCPU);
    A->set_requires_grad(true);
    B->set_requires_grad(true);
}

// A: uniform(+-sqrt(6 / (in + r))) from mt19937(42 + in + out); B: zeros.
static std::pair<TensorPtr, TensorPtr> new_pair(int in, int out, int rank) {
    auto A = zeros({in, rank}, kFloat32, kCPU);
    const float bound = std::sqrt(6.0f / (float)(in + rank));
    std::mt19937 gen(42 + in + out);
    std::uniform_real_distribution<float> dist(-bound, bound);
    float* a = A->data<float>();
    for (int64_t i = 0; i < A->numel(); ++i) a[i] = dist(gen);
    auto B = zeros({rank, out}, kFloat32, kCPU);
    A->set_requires_grad(true);
    B->set_requires_grad(true);
    return {A, B};
}

void LoraInjector::inject(GPT2Model& model, const LoraSpec& spec) {
    if (spec.rank <= 0) throw std::runtime_error("LoraInjector::inject: rank must be positive");
    model_ = &model;
    spec_ = spec;
    num_layers_ = model.config().n_layer;
    const int C = model.config().n_embd, r = spec.rank;
    const float scale = spec.alpha / (float)r;
    model.init_lora_modules();
    std::vector<int> layers = spec.layers;
    if (layers.empty())
        for (int i = 0; i < num_layers_; ++i) layers.push_back(i);
    int count = 0;
    for (int i : layers) {
        GPT2BlockWeights& b = model.get_block(i);
        for (LoraTarget t : spec.targets) {
            if (t == LoraTarget::AttnQKV) {
                if (spec.split_qkv) {
                    for (int part = 0; part < 3; ++part) {
                        auto ab = new_pair(C, C, r);
                        b.qkv_lin->attach_lora(ab.first, ab.second, scale, part * C, C);
                    }
                    count += 3;
                } else {
                    auto ab = new_pair(C, 3 * C, r);
                    b.qkv_lin->attach_lora(ab.first, ab.second, scale, 0, 3 * C);
                    ++count;
                }
            } else if (t == LoraTarget::AttnProj) {
                auto ab = new_pair(C, C, r);
                b.proj_lin->attach_lora(ab.first, ab.second, scale, 0, C);
                ++count;
            } else if (t == LoraTarget::MlpFcIn) {
                auto ab = new_pair(C, 4 * C, r);
                b.fc_in_lin->attach_lora(ab.first, ab.second, scale, 0, 4 * C);
                ++count;
            } else if (t == LoraTarget::MlpFcOut) {
                auto ab = new_pair(4 * C, C, r);
                b.fc_out_lin->attach_lora(ab.first, ab.second, scale, 0, C);
                ++count;
            }
        }
    }
    int64_t total = 0;
    const auto all = model.get_lora_parameters();
    for (const auto& p : all) total += p->numel();
    std::cout << "[LoraInjector] " << count << " adapters on " << layers.size() << " layers: rank " << r << ", alpha " << spec.alpha
              << ", " << total << " trainable values in " << all.size() << " tensors" << std::endl;
}

static void each_module(GPT2Model& model, void (LoRALinear::*fn)()) {
    for (int i = 0; i < model.config().n_layer; ++i) {
        GPT2BlockWeights& b = model.get_block(i);
        for (LoRALinear* m : {b.qkv_lin.get(), b.proj_lin.get(), b.fc_in_lin.get(), b.fc_out_lin.get()})
            if (m) (m->*fn)();
    }
}
void LoraInjector::merge_all(GPT2Model& model) { each_module(model, &LoRALinear::merge_to_base); }
void LoraInjector::unmerge_all(GPT2Model& model) { each_module(model, &LoRALinear::unmerge_from_base); }
void LoraInjector::merge() {
    if (merged_ || !model_) return;
    merge_all(*model_);
    merged_ = true;
}
void LoraInjector::unmerge() {
    if (!merged_ || !model_) return;
    unmerge_all(*model_);
    merged_ = false;
}

std::vector<TensorPtr> LoraInjector::collect_lora_parameters() const { return model_ ? model_->get_lora_parameters() : std::vector<TensorPtr>{}; }

std::vector<TensorPtr> LoraInjector::get_trainable_params() {
    auto params = collect_lora_parameters();
    for (auto& p : params) p->set_requires_grad(true);
    return params;
}

void LoraInjector::save_lora_safetensors(const std::string& path) const {
    if (!model_) throw std::runtime_error("LoraInjector::save_lora_safetensors: inject() was never called");
    LoraSaver::save_safetensors(path, *model_, spec_);
}

void LoraInjector::load_lora_safetensors(const std::string& path) {
    if (!model_) throw std::runtime_error("LoraInjector::load_lora_safetensors: inject() was never called");
    const LoRAState st = LoraSaver::load_safetensors(path);
    LoraSaver::attach_from_state(*model_, st);
    spec_.rank = st.rank; spec_.alpha = st.alpha; spec_.dropout = st.dropout; spec_.split_qkv = st.split_qkv;
    if (!st.targets.empty()) spec_.targets = st.targets;
}

void LoraInjector::print_info() const {
    std::cout << "[LoraInjector] rank " << spec_.rank << ", alpha " << spec_.alpha << ", dropout " << spec_.dropout << ", split_qkv "
              << (spec_.split_qkv ? "true" : "false") << ", layers " << num_layers_ << ", merged " << (merged_ ? "yes" : "no") << std::endl;
}

TensorPtr LoraInjector::lora_linear_forward(const TensorPtr& x, const TensorPtr& W, const TensorPtr& bias, const LoraState* lora, bool) {
    TensorPtr y = matmul(x, W);
    if (bias) y = add(y, bias);
    if (lora && lora->enabled) y = add(y, mul(matmul(matmul(x, lora->A), lora->B), lora->scale));
    return y;
}

}  // namespace ops
