#include "lm_loss.h"

#include <stdexcept>

#include "mft_cuda.h"
#include "../graph/engine_model.h"
#include "ops.h"

namespace ops {

using detail::check;
using detail::stream;

// The producer behind a model's forward() / forward_hidden() result, while nothing has forced the dense value yet.
static std::shared_ptr<detail::LazyLogits> deferred_model_output(const TensorPtr& t, bool hidden) {
    if (!t || !t->deferred()) return nullptr;
    auto ll = std::dynamic_pointer_cast<detail::LazyLogits>(t->deferred());
    return (ll && ll->hidden == hidden) ? ll : nullptr;
}

TensorPtr lm_cross_entropy(const TensorPtr& logits, const TensorPtr& labels, int ignore_index, const std::string& reduction) {
    if (!logits || !labels) throw std::runtime_error("lm_cross_entropy: null tensor");
    // Logits that a model's forward() handed out and nobody has read: run the fused lm head + loss (+ backward)
    // on the device, the [B,S,V] tensor is never formed (lm_cross_entropy core/lm_loss.cpp:268-382 on the values it
    // would hold).
    if (auto ll = deferred_model_output(logits, false))
        if (auto m = ll->model.lock()) return m->loss(ll->ids, ll->batch, ll->seq, labels, ignore_index, reduction);
    if (logits->dtype() != kFloat32 || labels->dtype() != kInt32) throw std::runtime_error("lm_cross_entropy: expects float32 logits and int32 labels");
    if (logits->shape().size() != 3 || labels->shape().size() != 2) throw std::runtime_error("lm_cross_entropy: expects logits [B,S,V] and labels [B,S]");
    if (reduction != "mean" && reduction != "sum") throw std::runtime_error("lm_cross_entropy: reduction must be 'mean' or 'sum' on this backend");
    const int64_t B = logits->shape()[0], S = logits->shape()[1], V = logits->shape()[2];
    if (labels->shape()[0] != B || labels->shape()[1] != S) throw std::runtime_error("lm_cross_entropy: labels shape mismatch");
    auto loss = std::make_shared<Tensor>(std::vector<int64_t>{1}, kFloat32, kCPU);
    auto n_valid = std::make_shared<Tensor>(std::vector<int64_t>{1}, kInt32, kCPU);
    auto lse = std::make_shared<Tensor>(std::vector<int64_t>{B * S}, kFloat32, kCPU);
    auto tgt = std::make_shared<Tensor>(std::vector<int64_t>{B * S}, kInt32, kCPU);
    auto acc = std::make_shared<Tensor>(std::vector<int64_t>{2}, kFloat32, kCPU);      // 8 bytes: one double
    auto status = std::make_shared<Tensor>(std::vector<int64_t>{1}, kInt32, kCPU);
    check(mft_ce_dense_fwd((const float*)logits->device_read(), (const int32_t*)labels->device_read(), B, S, V, ignore_index, (float*)loss->device_write(),
                           (int32_t*)n_valid->device_write(), (float*)lse->device_write(), (int32_t*)tgt->device_write(), (double*)acc->device_write(),
                           (int32_t*)status->device_readwrite(), stream()), "lm_cross_entropy");
    if (status->data<int32_t>()[0] != 0) throw std::runtime_error("lm_cross_entropy: label out of range");
    const int32_t n = n_valid->data<int32_t>()[0];
    const bool is_sum = reduction == "sum";
    if (is_sum) loss->data<float>()[0] = n > 0 ? loss->data<float>()[0] * (float)n : 0.0f;
    register_backward(loss, {logits}, std::make_shared<ClosureBackward>([logits, tgt, lse, n_valid, B, S, V, is_sum, n](const TensorPtr& g) {
        auto d = std::make_shared<Tensor>(logits->shape(), kFloat32, kCPU);
        const float outer = g ? g->data<float>()[0] : 1.0f;
        check(mft_ce_dense_bwd((const float*)logits->device_read(), (const int32_t*)tgt->device_read(), B, S, V, (const float*)lse->device_read(),
                               (const int32_t*)n_valid->device_read(), is_sum ? outer * (float)n : outer, (float*)d->device_write(), stream()),
              "lm_cross_entropy backward");
        return std::vector<TensorPtr>{d};
    }));
    return loss;
}

// bf16 compute type: the lm head and the shifted cross-entropy as one pass over vocabulary panels on the tensor cores
// (mft_lmhead_ce_fwd), the backward as a second pass that folds softmax - one_hot straight into dHidden
// (mft_lmhead_ce_bwd).  The [B,S,V] logits never reach memory, which is what the reference's streaming variant is
// for (core/lm_loss.cpp:384-481 forward, :165-266 backward).  The table W [V,H] is frozen here (no gradient).
static TensorPtr fused_lm_head_loss(const TensorPtr& hidden, const TensorPtr& W, const TensorPtr& labels, int ignore_index, bool is_sum) {
    const int64_t B = hidden->shape()[0], S = hidden->shape()[1], H = hidden->shape()[2], V = W->shape()[0];
    if (labels->shape()[0] != B || labels->shape()[1] != S) throw std::runtime_error("selected_token_lm_cross_entropy: labels shape mismatch");
    auto hb = detail::to_bf16(hidden), wb = detail::to_bf16(W);
    const int64_t ws_bytes = mft_lmhead_ce_workspace_bytes(B * S, H, V);
    auto ws = std::make_shared<Tensor>(std::vector<int64_t>{(ws_bytes + 3) / 4}, kFloat32, kCPU);
    auto loss = std::make_shared<Tensor>(std::vector<int64_t>{1}, kFloat32, kCPU);
    auto n_valid = std::make_shared<Tensor>(std::vector<int64_t>{1}, kInt32, kCPU);
    auto lse = std::make_shared<Tensor>(std::vector<int64_t>{B * S}, kFloat32, kCPU);
    auto status = std::make_shared<Tensor>(std::vector<int64_t>{1}, kInt32, kCPU);
    check(mft_lmhead_ce_fwd(hb->device_read(), wb->device_read(), (const int32_t*)labels->device_read(), B, S, H, V, ignore_index, (float*)loss->device_write(),
                            (int32_t*)n_valid->device_write(), (float*)lse->device_write(), (int32_t*)status->device_readwrite(), ws->device_write(), ws_bytes,
                            stream()), "streaming_lm_cross_entropy");
    if (status->data<int32_t>()[0] != 0) throw std::runtime_error("streaming_lm_cross_entropy: label out of range");
    const int32_t n = n_valid->data<int32_t>()[0];
    if (is_sum) loss->data<float>()[0] = n > 0 ? loss->data<float>()[0] * (float)n : 0.0f;
    register_backward(loss, {hidden}, std::make_shared<ClosureBackward>([=](const TensorPtr& g) {
        const int64_t ld_t = (V + 7) / 8 * 8;
        auto wt = std::make_shared<Tensor>(std::vector<int64_t>{H, ld_t}, kBFloat16, kCPU);
        check(mft_transpose_bf16_ld(wb->device_read(), wt->device_write(), V, H, ld_t, stream()), "streaming_lm_cross_entropy: table transpose");
        auto dh = std::make_shared<Tensor>(hidden->shape(), kBFloat16, kCPU);
        const float outer = g ? g->data<float>()[0] : 1.0f;
        check(mft_lmhead_ce_bwd(hb->device_read(), wb->device_read(), wt->device_read(), ld_t, (const int32_t*)labels->device_read(), B, S, H, V, ignore_index,
                                (const float*)lse->device_read(), (const int32_t*)n_valid->device_read(), 0, is_sum ? outer * (float)n : outer,
                                dh->device_write(), ws->device_write(), ws_bytes, stream()), "streaming_lm_cross_entropy backward");
        return std::vector<TensorPtr>{detail::bf16_to_f32(dh, hidden->shape())};
    }));
    return loss;
}

TensorPtr selected_token_lm_cross_entropy(const TensorPtr& hidden, const TensorPtr& W, const TensorPtr& labels, int ignore_index, const std::string& reduction) {
    if (!hidden || !W || !labels) throw std::runtime_error("selected_token_lm_cross_entropy: null tensor");
    // hidden states a model's forward_hidden() handed out, scored against that model's own (tied) table: fused path
    if (auto ll = deferred_model_output(hidden, true))
        if (auto m = ll->model.lock())
            if (W->shape().size() == 2 && W->shape()[0] == m->architecture().vocab && W->shape()[1] == m->architecture().hidden)
                return m->loss(ll->ids, ll->batch, ll->seq, labels, ignore_index, reduction);
    if (hidden->shape().size() != 3 || W->shape().size() != 2 || W->shape()[1] != hidden->shape()[2])
        throw std::runtime_error("selected_token_lm_cross_entropy: expects hidden [B,S,H] and weight [V,H]");
    if (detail::compute_bf16() && !W->requires_grad() && hidden->dtype() == kFloat32 && labels->dtype() == kInt32 && labels->shape().size() == 2 &&
        W->shape()[1] % 8 == 0 && (reduction == "mean" || reduction == "sum"))
        return fused_lm_head_loss(hidden, W, labels, ignore_index, reduction == "sum");
    // fp32 compute type: logits are formed by the fp32 matmul so that loss and gradients keep fp32 accuracy
    return lm_cross_entropy(matmul_rhs_T(hidden, W), labels, ignore_index, reduction);
}
TensorPtr streaming_lm_cross_entropy(const TensorPtr& hidden, const TensorPtr& W, const TensorPtr& labels, int ignore_index, const std::string& reduction) {
    return selected_token_lm_cross_entropy(hidden, W, labels, ignore_index, reduction);
}

}  // namespace ops
