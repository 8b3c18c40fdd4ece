// What the three model classes (GPT2Model, QwenModel, GemmaModel) share: the bridge from host-visible weight and
// adapter tensors to the device step engine of include/mft_step.h.
//
// A model class keeps its weights as ops::Tensor objects exactly as the reference's classes do (callers fill them
// through data<T>(), replace them with assign_weight, attach adapters through LoRALinear).  forward() does not run a
// layer-by-layer operator graph.  It brings the engine up to date with those tensors and returns the logits as a
// DEFERRED tensor: lm_cross_entropy recognises it and runs the fused forward + loss (+ backward) kernels, so the
// [B,S,V] logits never exist; any other access computes them on demand.
//
//  * frozen weights: re-uploaded when a tensor object was replaced or a mutable host pointer to it was taken since
//    the last upload (a caller that keeps an old pointer and writes through it later is not seen);
//  * adapters: the A/B tensors found on the model's LoRALinear modules are BOUND to their slices of the engine's flat
//    f32 parameter bucket, their gradients to slices of a flat accumulation bucket, so ops::Adam and
//    Optimizer::clip_grad_norm work on that memory directly and nothing is copied per step;
//  * gradients accumulate across backward() calls until zero_grad, and honour the gradient that reaches the loss
//    (a loss scaled by 1/accumulation_steps before backward()).
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "mft_step.h"
#include "../core/tensor.h"
#include "../nn/lora_linear.h"

namespace ops {
namespace detail {

class EngineModel : public std::enable_shared_from_this<EngineModel> {
public:
    using ParamsFn = std::function<std::vector<TensorPtr>()>;                 // the engine's parameter order
    using ModuleFn = std::function<LoRALinear*(int layer, uint32_t target)>;  // MFT_LORA_* bit -> module (or null)

    EngineModel(const mft_model_config_t& architecture, ParamsFn params, ModuleFn modules);
    ~EngineModel();
    EngineModel(const EngineModel&) = delete;
    EngineModel& operator=(const EngineModel&) = delete;

    // input_ids int32 [B,S]; attention_mask (may be null) [B,S] with ones first, then zeros: positions after the
    // first zero are padding, which a causal model's scored positions never see.  Any other pattern is refused.
    TensorPtr forward(const TensorPtr& input_ids, const TensorPtr& attention_mask);
    // Same, but the deferred value is the final-norm output [B,S,hidden] (QwenModel::forward_hidden); the loss
    // functions that take (hidden, lm-head weight) recognise it.
    TensorPtr forward_hidden(const TensorPtr& input_ids, const TensorPtr& attention_mask);
    // logits = hidden . table^T for a deferred hidden state of this model (stays deferred); null otherwise.
    TensorPtr lm_head_of(const TensorPtr& hidden);
    // Adapter tensors in the reference's get_lora_parameters() order (A then B per module).
    std::vector<TensorPtr> lora_parameters() const;
    const mft_model_config_t& architecture() const { return arch_; }
    // Hint for the first engine construction (tokens per call the caller expects at most).
    void reserve(int batch, int seq);

    // Used by lm_cross_entropy on a deferred logits tensor.
    TensorPtr loss(const std::vector<int32_t>& ids, int batch, int seq, const TensorPtr& labels, int ignore_index, const std::string& reduction);
    void logits_into(const std::vector<int32_t>& ids, int batch, int seq, Tensor& out);
    void hidden_into(const std::vector<int32_t>& ids, int batch, int seq, Tensor& out);

private:
    struct Signature {
        uint32_t mask = 0;
        int rank = 0;
        float alpha = 0.f;
        bool operator==(const Signature& o) const { return mask == o.mask && rank == o.rank && alpha == o.alpha; }
    };
    mft_model_config_t arch_;
    ParamsFn params_fn_;
    ModuleFn module_fn_;
    mft_model_t* engine_ = nullptr;
    Signature sig_;
    int cap_tokens_ = 0, cap_seq_ = 0;
    std::vector<const Tensor*> seen_ptr_;
    std::vector<uint64_t> seen_writes_;
    // adapters
    float *p_bucket_ = nullptr, *g_step_ = nullptr, *g_acc_ = nullptr;   // engine params, engine per-call grads, accumulated grads
    int64_t bucket_n_ = 0;
    std::vector<int64_t> offsets_;
    std::vector<bool> has_grad_;
    std::vector<TensorPtr> grads_;                 // bound to g_acc_ slices
    std::vector<std::weak_ptr<Tensor>> bound_;     // adapter tensors bound to p_bucket_ slices

    Signature scan(std::vector<TensorPtr>* tensors) const;
    void ensure(int batch, int seq);
    void rebuild(const Signature& sig);
    void release_engine();
    void sync_parameters();
    void sync_adapters();
    void accumulate(float upstream);
    TensorPtr deferred_output(const TensorPtr& input_ids, const TensorPtr& attention_mask, bool hidden);
};

// The deferred value behind the logits a model's forward() returns.
class LazyLogits : public Deferred {
public:
    LazyLogits(std::weak_ptr<EngineModel> m, std::vector<int32_t> ids, int batch, int seq, bool hidden = false)
        : model(std::move(m)), ids(std::move(ids)), batch(batch), seq(seq), hidden(hidden) {}
    void materialize(Tensor& into) override;
    std::weak_ptr<EngineModel> model;
    std::vector<int32_t> ids;
    int batch, seq;
    bool hidden;            // the value is the final hidden state, not the logits
};

// Engine order of the adapter targets inside one layer, per family (the reference's get_lora_parameters() orders:
// gpt2_model.cpp:221-241, qwen_model.cpp:186-205, gemma_model.cpp:736-757).
const std::vector<uint32_t>& lora_target_order(int family);

}  // namespace detail
}  // namespace ops
