#include "memory_efficient_attention.h"

#include <cmath>

#include "mft_cuda.h"
#include "ops.h"

namespace ops {

using detail::check;
using detail::stream;

namespace {

// True when `mask` holds the causal pattern of create_causal_mask for S positions: 0 on and below the diagonal,
// a large negative number above it ([S,S], with any number of leading 1-dimensions).
bool is_plain_causal_mask(const TensorPtr& mask, int64_t S) {
    if (!mask || mask->dtype() != kFloat32 || mask->numel() != S * S) return false;
    const auto& sh = mask->shape();
    if (sh.size() < 2 || sh[sh.size() - 1] != S || sh[sh.size() - 2] != S) return false;
    const float* m = static_cast<const Tensor&>(*mask).data<float>();
    for (int64_t i = 0; i < S; ++i)
        for (int64_t j = 0; j < S; ++j) {
            const float v = m[i * S + j];
            if (j <= i ? v != 0.0f : !(v <= -1e4f)) return false;
        }
    return true;
}

// Fused flash-style attention on [B, heads, S, head_dim] tensors: one kernel forward, the recomputing backward
// kernels for dQ / dK / dV; the [S,S] scores never reach memory (the purpose of memory_efficient_attention,
// core/memory_efficient_attention.cpp:33-238 of the reference, which tiles the same computation on the host).
TensorPtr fused_causal_attention(const TensorPtr& q, const TensorPtr& k, const TensorPtr& v, float scale) {
    const auto& sh = q->shape();
    const int64_t B = sh[0], H = sh[1], S = sh[2], hd = sh[3], Hkv = k->shape()[1];
    auto qb = detail::to_bf16(q), kb = detail::to_bf16(k), vb = detail::to_bf16(v);
    auto ob = std::make_shared<Tensor>(sh, kBFloat16, kCPU);
    auto lse = std::make_shared<Tensor>(std::vector<int64_t>{B, H, S}, kFloat32, kCPU);
    const mft_strides_t sq{H * S * hd, hd, S * hd}, skv{Hkv * S * hd, hd, S * hd};
    check(mft_attn_fwd(qb->device_read(), sq, kb->device_read(), skv, vb->device_read(), skv, ob->device_write(), sq, (float*)lse->device_write(),
                       B, S, H, Hkv, hd, scale, 0, stream()), "memory_efficient_attention");
    auto out = detail::bf16_to_f32(ob, sh);
    register_backward(out, {q, k, v}, std::make_shared<ClosureBackward>([=](const TensorPtr& g) {
        auto gb = detail::to_bf16(g);
        auto dq = std::make_shared<Tensor>(q->shape(), kBFloat16, kCPU);
        auto dk = std::make_shared<Tensor>(k->shape(), kBFloat16, kCPU);
        auto dv = std::make_shared<Tensor>(v->shape(), kBFloat16, kCPU);
        auto delta = std::make_shared<Tensor>(std::vector<int64_t>{B, H, S}, kFloat32, kCPU);
        auto acc = std::make_shared<Tensor>(std::vector<int64_t>{2 * B * S * Hkv * hd}, kFloat32, kCPU);
        check(mft_attn_bwd(qb->device_read(), sq, kb->device_read(), skv, vb->device_read(), skv, ob->device_read(), sq, gb->device_read(), sq,
                           (const float*)lse->device_read(), dq->device_write(), dk->device_write(), dv->device_write(), (float*)delta->device_write(),
                           (float*)acc->device_write(), B, S, H, Hkv, hd, scale, 0, stream()), "memory_efficient_attention backward");
        return std::vector<TensorPtr>{detail::bf16_to_f32(dq, q->shape()), detail::bf16_to_f32(dk, k->shape()), detail::bf16_to_f32(dv, v->shape())};
    }));
    return out;
}

}  // namespace

TensorPtr memory_efficient_attention(const TensorPtr& q, const TensorPtr& k, const TensorPtr& v, const TensorPtr& causal_mask,
                                     const MemoryEfficientAttentionConfig& config) {
    if (!q || !k || !v || q->shape().size() != 4) throw TensorError("memory_efficient_attention: expects [B,heads,S,head_dim] tensors");
    const int64_t S = q->shape()[2], hd = q->shape()[3];
    const float scale = config.scale > 0.f ? config.scale : 1.0f / std::sqrt((float)hd);
    // bf16 compute type: the fused kernels, when the mask is the causal one (given or implied) and the shapes are
    // ones the kernels take (KV heads dividing the query heads, even head_dim <= 256)
    if (detail::compute_bf16() && k->shape() == v->shape() && k->shape().size() == 4 && k->shape()[0] == q->shape()[0] && k->shape()[2] == S &&
        k->shape()[3] == hd && k->shape()[1] > 0 && q->shape()[1] % k->shape()[1] == 0 && hd % 2 == 0 && hd <= 256 &&
        q->dtype() == kFloat32 && k->dtype() == kFloat32 && v->dtype() == kFloat32 &&
        (causal_mask ? is_plain_causal_mask(causal_mask, S) : config.use_causal_mask))
        return fused_causal_attention(q, k, v, scale);
    // fp32 compute type (and masks other than the causal one): composed from the fp32 operators
    auto scores = mul(matmul(q, transpose(k, 2, 3)), scale);
    TensorPtr mask = causal_mask;
    if (!mask && config.use_causal_mask) mask = create_causal_mask((int)S);
    if (mask) scores = add(scores, mask);
    return matmul(softmax(scores, -1), v);
}

}  // namespace ops
