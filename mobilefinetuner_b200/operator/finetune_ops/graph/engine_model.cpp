#include "engine_model.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

#include "mft_cuda.h"
#include "../core/autograd_engine.h"

namespace ops {
namespace detail {

namespace {
void ok(int32_t s, const char* what) {
    if (s != MFT_OK) throw std::runtime_error(std::string(what) + ": " + mft_last_error());
}
// f32 view of a weight tensor on the host (frozen weights may be stored as bf16 / f16)
const float* host_f32(const TensorPtr& t, TensorPtr& keep) {
    if (t->dtype() == kFloat32) return static_cast<const Tensor&>(*t).data<float>();
    keep = cast(t, kFloat32);
    return static_cast<const Tensor&>(*keep).data<float>();
}
bool all_zero(const TensorPtr& t) {
    const float* p = static_cast<const Tensor&>(*t).data<float>();
    for (int64_t i = 0; i < t->numel(); ++i)
        if (p[i] != 0.0f) return false;
    return true;
}
}  // namespace

const std::vector<uint32_t>& lora_target_order(int family) {
    static const std::vector<uint32_t> gpt2 = {MFT_LORA_Q, MFT_LORA_O, MFT_LORA_GATE, MFT_LORA_DOWN};      // c_attn, c_proj, c_fc, mlp c_proj
    static const std::vector<uint32_t> qwen = {MFT_LORA_Q, MFT_LORA_V, MFT_LORA_K, MFT_LORA_O};
    static const std::vector<uint32_t> gemma = {MFT_LORA_Q, MFT_LORA_K, MFT_LORA_V, MFT_LORA_O, MFT_LORA_GATE, MFT_LORA_UP, MFT_LORA_DOWN};
    return family == MFT_FAMILY_GPT2 ? gpt2 : family == MFT_FAMILY_QWEN ? qwen : gemma;
}

EngineModel::EngineModel(const mft_model_config_t& a, ParamsFn p, ModuleFn m) : arch_(a), params_fn_(std::move(p)), module_fn_(std::move(m)) {
    arch_.lora_rank = 0;
    arch_.lora_alpha = 0.f;
    arch_.lora_targets = 0;
}

EngineModel::~EngineModel() {
    try { release_engine(); } catch (...) {}
}

void EngineModel::reserve(int batch, int seq) {
    cap_tokens_ = std::max(cap_tokens_, batch * seq);
    cap_seq_ = std::max(cap_seq_, seq);
}

// Which adapters are attached, and with which rank / scale.  The engine applies one selection to every layer.
EngineModel::Signature EngineModel::scan(std::vector<TensorPtr>* tensors) const {
    Signature sig;
    bool first_layer = true;
    const bool peft_layout = arch_.family == MFT_FAMILY_GEMMA;       // A [r,in], B [out,r]
    for (int l = 0; l < arch_.layers; ++l) {
        uint32_t mask = 0;
        for (uint32_t bit : lora_target_order(arch_.family)) {
            LoRALinear* mod = module_fn_(l, bit);
            if (!mod || mod->is_merged()) continue;
            const int64_t in = mod->W()->shape()[0], out = mod->W()->shape()[1];
            const LoRASlice* full = nullptr;
            for (const LoRASlice& s : mod->slices()) {
                if (s.col0 == 0 && (s.cols < 0 || s.cols == out)) {
                    if (full) throw std::runtime_error("device engine: more than one full-width adapter on one linear is not supported");
                    full = &s;
                } else if (!all_zero(s.B)) {
                    // Adapters that cover part of the columns only add to the forward value and never train
                    // (nn/lora_linear.cpp:442-459); with B = 0, their initial value, they contribute exactly nothing.
                    throw std::runtime_error("device engine: a partial-column adapter with non-zero B is not supported (use split_qkv = false)");
                }
            }
            if (!full) continue;
            const auto& sa = full->A->shape();
            const auto& sb = full->B->shape();
            if (sa.size() != 2 || sb.size() != 2) throw std::runtime_error("device engine: adapter tensors must be 2-D");
            const int64_t r = peft_layout ? sa[0] : sa[1];
            const bool shape_ok = peft_layout ? (sa[1] == in && sb[0] == out && sb[1] == r) : (sa[0] == in && sb[0] == r && sb[1] == out);
            if (!shape_ok || r <= 0 || r > 64) throw std::runtime_error("device engine: adapter shapes do not match this family's layout (or rank > 64)");
            const float alpha = full->scale * (float)r;
            if (sig.rank == 0) { sig.rank = (int)r; sig.alpha = alpha; }
            else if (sig.rank != r || std::fabs(sig.alpha - alpha) > 1e-6f * std::fabs(alpha))
                throw std::runtime_error("device engine: all adapters must share one rank and one alpha");
            mask |= bit;
            if (tensors) { tensors->push_back(full->A); tensors->push_back(full->B); }
        }
        if (first_layer) { sig.mask = mask; first_layer = false; }
        else if (mask != sig.mask) throw std::runtime_error("device engine: every layer must carry the same set of adapters");
    }
    if (sig.mask == 0) sig = Signature();
    return sig;
}

std::vector<TensorPtr> EngineModel::lora_parameters() const {
    // every trainable tensor of every module, in the family's order (also partial-column slices, as the reference lists them)
    std::vector<TensorPtr> out;
    for (int l = 0; l < arch_.layers; ++l)
        for (uint32_t bit : lora_target_order(arch_.family))
            if (LoRALinear* mod = module_fn_(l, bit)) {
                auto p = mod->trainable_parameters();
                out.insert(out.end(), p.begin(), p.end());
            }
    return out;
}

void EngineModel::release_engine() {
    for (auto& w : bound_)
        if (auto t = w.lock()) t->unbind_device();
    bound_.clear();
    for (auto& g : grads_)
        if (g) g->unbind_device();
    grads_.clear();
    if (g_acc_) { mft_free(g_acc_, detail::stream()); g_acc_ = nullptr; }
    if (engine_) { mft_model_destroy(engine_); engine_ = nullptr; }
    p_bucket_ = g_step_ = nullptr;
    bucket_n_ = 0;
    offsets_.clear();
    has_grad_.clear();
    seen_ptr_.clear();
    seen_writes_.clear();
}

void EngineModel::rebuild(const Signature& sig) {
    release_engine();
    detail::ensure_runtime();
    mft_model_config_t cfg = arch_;
    cfg.lora_rank = sig.rank;
    cfg.lora_alpha = sig.alpha;
    cfg.lora_targets = sig.mask;
    cfg.max_seq = std::max(cap_seq_, 8);
    cfg.max_batch = std::max(1, (cap_tokens_ + cfg.max_seq - 1) / cfg.max_seq);
    ok(mft_model_create(&cfg, detail::stream(), &engine_), "mft_model_create");
    sig_ = sig;
    const int n = mft_model_lora_count(engine_);
    if (n > 0) {
        ok(mft_model_buckets(engine_, &p_bucket_, &g_step_, &bucket_n_), "mft_model_buckets");
        void* p = nullptr;
        ok(mft_malloc((size_t)bucket_n_ * 4, detail::stream(), &p), "gradient accumulation bucket");
        g_acc_ = static_cast<float*>(p);
        ok(mft_memset(g_acc_, 0, (size_t)bucket_n_ * 4, detail::stream()), "memset");
        offsets_.resize(n);
        has_grad_.resize(n);
        grads_.assign(n, nullptr);
        for (int i = 0; i < n; ++i) {
            ok(mft_model_lora_offset(engine_, i, &offsets_[i]), "mft_model_lora_offset");
            has_grad_[i] = mft_model_lora_has_grad(engine_, i) != 0;
        }
    }
}

void EngineModel::ensure(int batch, int seq) {
    const Signature sig = scan(nullptr);
    const bool too_small = batch * seq > cap_tokens_ || seq > cap_seq_;
    reserve(batch, seq);
    if (!engine_ || too_small || !(sig == sig_)) rebuild(sig);
}

void EngineModel::sync_parameters() {
    const std::vector<TensorPtr> params = params_fn_();
    const int n = mft_model_param_count(engine_);
    if ((int)params.size() != n) throw std::runtime_error("device engine: parameters() does not match the architecture");
    if (seen_ptr_.size() != (size_t)n) { seen_ptr_.assign(n, nullptr); seen_writes_.assign(n, 0); }
    for (int i = 0; i < n; ++i) {
        const TensorPtr& t = params[i];
        if (!t) throw std::runtime_error("device engine: parameter " + std::to_string(i) + " is null");
        if (seen_ptr_[i] == t.get() && seen_writes_[i] == t->host_write_count()) continue;
        int64_t r = 0, c = 0;
        ok(mft_model_param_shape(engine_, i, &r, &c), "mft_model_param_shape");
        if (t->numel() != r * c) throw std::runtime_error("device engine: parameter " + std::to_string(i) + " has the wrong size");
        TensorPtr keep;
        ok(mft_model_set_param_host(engine_, i, host_f32(t, keep)), "mft_model_set_param_host");
        seen_ptr_[i] = t.get();
        seen_writes_[i] = t->host_write_count();
    }
}

void EngineModel::sync_adapters() {
    if (bucket_n_ == 0) return;
    std::vector<TensorPtr> tensors;
    scan(&tensors);
    if (tensors.size() != offsets_.size()) throw std::runtime_error("device engine: adapter list changed under the engine");
    bound_.clear();
    for (size_t i = 0; i < tensors.size(); ++i) {
        const TensorPtr& t = tensors[i];
        int64_t r = 0, c = 0;
        ok(mft_model_lora_shape(engine_, (int)i, &r, &c), "mft_model_lora_shape");
        if (t->dtype() != kFloat32 || t->shape().size() != 2 || t->shape()[0] != r || t->shape()[1] != c)
            throw std::runtime_error("device engine: adapter tensor " + std::to_string(i) + " has the wrong shape or type");
        float* home = p_bucket_ + offsets_[i];
        if (t->bound_device() != home) t->bind_device(home);        // moves the current value into the bucket
        else if (t->host_dirty()) t->device_read();                  // host writes since the last kernel: upload
        t->set_requires_grad(true);
        bound_.push_back(t);
    }
    // ops::Adam updates the bucket memory through the tensors: always re-pack the bf16 panels the GEMMs read
    ok(mft_model_mark_lora_dirty(engine_), "mft_model_mark_lora_dirty");
}

TensorPtr EngineModel::forward(const TensorPtr& ids, const TensorPtr& mask) { return deferred_output(ids, mask, false); }
TensorPtr EngineModel::forward_hidden(const TensorPtr& ids, const TensorPtr& mask) { return deferred_output(ids, mask, true); }

TensorPtr EngineModel::lm_head_of(const TensorPtr& hidden) {
    if (!hidden || !hidden->deferred()) return nullptr;
    auto ll = std::dynamic_pointer_cast<LazyLogits>(hidden->deferred());
    if (!ll || !ll->hidden || ll->model.lock().get() != this) return nullptr;
    auto producer = std::make_shared<LazyLogits>(weak_from_this(), ll->ids, ll->batch, ll->seq, false);
    return Tensor::make_deferred({ll->batch, ll->seq, arch_.vocab}, kFloat32, producer);
}

TensorPtr EngineModel::deferred_output(const TensorPtr& ids, const TensorPtr& mask, bool hidden) {
    if (!ids || ids->dtype() != kInt32 || ids->shape().size() != 2) throw std::runtime_error("forward: input_ids must be int32 [batch, seq]");
    const int B = (int)ids->shape()[0], S = (int)ids->shape()[1];
    if (S < 2) throw std::runtime_error("forward: the device engine needs at least two positions per sequence");
    if (mask) {
        if (mask->numel() != (int64_t)B * S) throw std::runtime_error("forward: attention_mask shape mismatch");
        const bool as_int = mask->dtype() == kInt32;
        if (!as_int && mask->dtype() != kFloat32) throw std::runtime_error("forward: attention_mask must be int32 or float32");
        const void* p = static_cast<const Tensor&>(*mask).data_ptr();
        for (int b = 0; b < B; ++b) {
            bool pad = false;
            for (int s = 0; s < S; ++s) {
                const bool one = as_int ? static_cast<const int32_t*>(p)[b * S + s] != 0 : static_cast<const float*>(p)[b * S + s] != 0.0f;
                if (!one) pad = true;
                else if (pad)
                    throw std::runtime_error("forward: only right-padded attention masks are supported (valid positions first); "
                                             "a causal model's scored positions never attend to right padding, so it needs no mask");
            }
        }
    }
    ensure(B, S);
    sync_parameters();
    sync_adapters();
    const int32_t* src = static_cast<const Tensor&>(*ids).data<int32_t>();
    std::vector<int32_t> copy(src, src + (size_t)B * S);
    auto producer = std::make_shared<LazyLogits>(weak_from_this(), std::move(copy), B, S, hidden);
    return Tensor::make_deferred({B, S, hidden ? arch_.hidden : arch_.vocab}, kFloat32, producer);
}

void LazyLogits::materialize(Tensor& into) {
    auto m = model.lock();
    if (!m) throw std::runtime_error("logits: the model that produced them no longer exists");
    if (hidden) m->hidden_into(ids, batch, seq, into);
    else m->logits_into(ids, batch, seq, into);
}

void EngineModel::hidden_into(const std::vector<int32_t>& ids, int B, int S, Tensor& out) {
    ensure(B, S);
    sync_parameters();
    sync_adapters();
    ok(mft_model_forward_hidden(engine_, ids.data(), B, S, static_cast<float*>(out.device_write())), "mft_model_forward_hidden");
}

void EngineModel::logits_into(const std::vector<int32_t>& ids, int B, int S, Tensor& out) {
    ensure(B, S);
    sync_parameters();
    sync_adapters();
    ok(mft_model_forward_logits(engine_, ids.data(), B, S, static_cast<float*>(out.device_write())), "mft_model_forward_logits");
}

void EngineModel::accumulate(float upstream) {
    // param.grad += upstream * (gradient of this call); gradients live in one flat bucket the tensors are bound to
    std::vector<TensorPtr> tensors;
    scan(&tensors);
    for (size_t i = 0; i < tensors.size() && i < grads_.size(); ++i) {
        if (!has_grad_[i]) continue;                       // the reference delivers no gradient here: grad() stays null
        if (!grads_[i]) {
            grads_[i] = std::make_shared<Tensor>(tensors[i]->shape(), kFloat32, kCPU);
            grads_[i]->bind_device(g_acc_ + offsets_[i]);
        }
        if (tensors[i]->grad() != grads_[i]) {
            // first gradient since the caller dropped or replaced it: start from zero
            ok(mft_memset(g_acc_ + offsets_[i], 0, grads_[i]->nbytes(), detail::stream()), "memset");
            grads_[i]->device_write();
            tensors[i]->set_grad(grads_[i]);
        } else {
            grads_[i]->device_readwrite();                  // host edits (a clip done on the host) go up first
        }
    }
    if (upstream != 1.0f) ok(mft_scale_f32(g_step_, upstream, bucket_n_, detail::stream()), "scale");
    ok(mft_add_f32(g_acc_, g_step_, g_acc_, bucket_n_, detail::stream()), "accumulate");
}

TensorPtr EngineModel::loss(const std::vector<int32_t>& ids, int B, int S, const TensorPtr& labels, int ignore_index, const std::string& reduction) {
    if (!labels || labels->dtype() != kInt32 || labels->numel() != (int64_t)B * S) throw std::runtime_error("lm_cross_entropy: labels must be int32 [batch, seq]");
    if (reduction != "mean" && reduction != "sum") throw std::runtime_error("lm_cross_entropy: reduction must be 'mean' or 'sum' on this backend");
    ensure(B, S);
    sync_parameters();
    sync_adapters();
    const int32_t* lab = static_cast<const Tensor&>(*labels).data<int32_t>();
    std::vector<int32_t> remapped;
    if (ignore_index != -100) {                               // the engine's ignore value is -100
        remapped.assign(lab, lab + (size_t)B * S);
        for (auto& v : remapped) v = v == ignore_index ? -100 : v;
        lab = remapped.data();
    }
    int64_t n_valid = 0;
    for (int b = 0; b < B; ++b)
        for (int s = 1; s < S; ++s) n_valid += lab[b * S + s] != -100;
    const bool sum = reduction == "sum";
    bool trainable = false;
    for (size_t i = 0; i < has_grad_.size(); ++i) trainable = trainable || has_grad_[i];
    auto out = std::make_shared<Tensor>(std::vector<int64_t>{1}, kFloat32, kCPU);
    float value = 0.f;
    if (autograd::Engine::instance().is_enabled() && trainable) {
        int32_t nv = 0;
        ok(mft_model_zero_grad(engine_), "mft_model_zero_grad");
        ok(mft_model_forward_backward(engine_, ids.data(), lab, B, S, 0, &value, &nv), "mft_model_forward_backward");
        std::weak_ptr<EngineModel> self = weak_from_this();
        const float factor = sum ? (float)n_valid : 1.0f;
        auto fn = std::make_shared<ClosureBackward>([self, factor](const TensorPtr& g) {
            if (auto m = self.lock()) m->accumulate((g ? static_cast<const Tensor&>(*g).data<float>()[0] : 1.0f) * factor);
            return std::vector<TensorPtr>{};
        });
        autograd::Engine::instance().register_node(out, {}, fn);
    } else {
        ok(mft_model_forward_loss(engine_, ids.data(), lab, B, S, &value), "mft_model_forward_loss");
    }
    out->data<float>()[0] = sum ? (n_valid > 0 ? value * (float)n_valid : 0.0f) : value;
    return out;
}

}  // namespace detail
}  // namespace ops
