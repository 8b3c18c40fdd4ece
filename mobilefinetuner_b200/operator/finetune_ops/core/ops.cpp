// Eager operators of namespace ops on device-resident tensors.  Forward and
// backward of every operator are kernel launches through the C ABI
// (include/mft_cuda.h); nothing is computed on the host except shape logic and
// a few dtype conversions of frozen weights.
#include "ops.h"

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <stdexcept>

#include "mft_cuda.h"
#include "autograd_engine.h"

namespace ops {

using detail::check;
using detail::stream;

// ---------------------------------------------------------------- compute type of the eager operators
static std::atomic<int>& compute_dtype_slot() {
    static std::atomic<int> v([] {
        const char* e = std::getenv("MFT_COMPUTE_DTYPE");
        const std::string s = e ? e : "";
        return (s == "bf16" || s == "bfloat16" || s == "BF16") ? (int)kBFloat16 : (int)kFloat32;
    }());
    return v;
}
void set_compute_dtype(DType dtype) {
    if (dtype != kFloat32 && dtype != kBFloat16) throw TensorError("set_compute_dtype: float32 or bfloat16");
    compute_dtype_slot().store((int)dtype);
}
DType compute_dtype() { return (DType)compute_dtype_slot().load(); }

namespace detail {
bool compute_bf16() { return compute_dtype() == kBFloat16; }
TensorPtr to_bf16(const TensorPtr& t) {
    if (t->dtype() == kBFloat16) return t;
    if (t->dtype() != kFloat32) throw TensorError("to_bf16: float32 or bfloat16 tensor expected");
    auto out = std::make_shared<Tensor>(t->shape(), kBFloat16, kCPU);
    check(mft_cast_f32_to_bf16((const float*)t->device_read(), out->device_write(), t->numel(), stream()), "cast to bf16");
    return out;
}
TensorPtr bf16_to_f32(const TensorPtr& t, const std::vector<int64_t>& shape) {
    auto out = std::make_shared<Tensor>(shape, kFloat32, kCPU);
    if (out->numel() != t->numel()) throw TensorError("bf16_to_f32: element count mismatch");
    check(mft_cast_bf16_to_f32(t->device_read(), (float*)out->device_write(), t->numel(), stream()), "cast to f32");
    return out;
}
}  // namespace detail

namespace {

TensorPtr make(const std::vector<int64_t>& shape) { return std::make_shared<Tensor>(shape, kFloat32, kCPU); }

void require_f32(const TensorPtr& t, const char* who) {
    if (!t) throw TensorError(std::string(who) + ": null tensor");
    if (t->dtype() != kFloat32) throw TensorError(std::string(who) + ": float32 tensor expected");
}

int64_t prod(const std::vector<int64_t>& s, size_t from, size_t to) {
    int64_t n = 1;
    for (size_t i = from; i < to; ++i) n *= s[i];
    return n;
}

BackwardFunctionPtr closure(ClosureBackward::Fn fn) { return std::make_shared<ClosureBackward>(std::move(fn)); }

// Reduce a broadcast gradient back to `shape` (sum over the broadcast dimensions).
TensorPtr sum_to_shape(const TensorPtr& g, const std::vector<int64_t>& shape) {
    if (g->shape() == shape) return g;
    TensorPtr cur = g;
    std::vector<int64_t> gs = g->shape();
    const size_t lead = gs.size() - shape.size();
    // leading extra dims: fold them into one reduction
    if (lead > 0) {
        const int64_t outer = prod(gs, 0, lead), inner = prod(gs, lead, gs.size());
        auto r = make(std::vector<int64_t>(gs.begin() + (long)lead, gs.end()));
        check(mft_reduce_sum_f32((const float*)cur->device_read(), (float*)r->device_write(), 1, outer, inner, 1.0f, stream()), "sum_to_shape");
        cur = r;
        gs = cur->shape();
    }
    for (size_t d = 0; d < shape.size(); ++d) {
        if (shape[d] == 1 && gs[d] != 1) {
            const int64_t outer = prod(gs, 0, d), red = gs[d], inner = prod(gs, d + 1, gs.size());
            gs[d] = 1;
            auto r = make(gs);
            check(mft_reduce_sum_f32((const float*)cur->device_read(), (float*)r->device_write(), outer, red, inner, 1.0f, stream()), "sum_to_shape");
            cur = r;
        }
    }
    return cur;
}

TensorPtr binary(int op, const TensorPtr& a, const TensorPtr& b) {
    require_f32(a, "elementwise op"); require_f32(b, "elementwise op");
    const auto shape = broadcast_shape(a, b);
    auto out = make(shape);
    check(mft_ew_binary_f32(op, (const float*)a->device_read(), a->shape().data(), (int)a->shape().size(), (const float*)b->device_read(),
                            b->shape().data(), (int)b->shape().size(), (float*)out->device_write(), shape.data(), (int)shape.size(), stream()),
          "elementwise op");
    return out;
}
TensorPtr scalar_op(int op, const TensorPtr& a, float s, bool scalar_first) {
    require_f32(a, "scalar op");
    auto out = make(a->shape());
    check(mft_ew_scalar_f32(op, (const float*)a->device_read(), s, scalar_first ? 1 : 0, (float*)out->device_write(), a->numel(), stream()), "scalar op");
    return out;
}
TensorPtr unary(int op, const TensorPtr& a, float p = 0.f) {
    require_f32(a, "unary op");
    auto out = make(a->shape());
    check(mft_ew_unary_f32(op, (const float*)a->device_read(), p, (float*)out->device_write(), a->numel(), stream()), "unary op");
    return out;
}

TensorPtr permute_raw(const TensorPtr& t, const std::vector<int>& dims) {
    const int nd = (int)t->shape().size();
    if ((int)dims.size() != nd) throw TensorError("permute: rank mismatch");
    if (DTypeUtils::size_of(t->dtype()) != 4) throw TensorError("permute: 32-bit element types only");
    std::vector<int64_t> shape((size_t)nd);
    std::vector<int32_t> perm((size_t)nd);
    for (int k = 0; k < nd; ++k) { perm[(size_t)k] = dims[(size_t)k] < 0 ? dims[(size_t)k] + nd : dims[(size_t)k]; shape[(size_t)k] = t->shape()[(size_t)perm[(size_t)k]]; }
    auto out = std::make_shared<Tensor>(shape, t->dtype(), t->device());
    check(mft_permute_b32(t->device_read(), out->device_write(), t->shape().data(), perm.data(), nd, stream()), "permute");
    return out;
}

TensorPtr as_f32(const TensorPtr& t) { return t->dtype() == kFloat32 ? t : ops::cast(t, kFloat32); }

// C = A x B (or A x B^T): A [..,M,K]; B 2-D (shared by every batch) or with the same leading dims.
TensorPtr matmul_raw(const TensorPtr& a, const TensorPtr& b_in, bool trans_b) {
    require_f32(a, "matmul");
    TensorPtr b = as_f32(b_in);
    const auto& as = a->shape();
    const auto& bs = b->shape();
    if (as.size() < 1 || bs.size() < 2) throw TensorError("matmul: operands need at least 2 dimensions");
    const int64_t K = as.back();
    const int64_t M = as.size() >= 2 ? as[as.size() - 2] : 1;
    const int64_t bk = trans_b ? bs.back() : bs[bs.size() - 2];
    const int64_t N = trans_b ? bs[bs.size() - 2] : bs.back();
    if (bk != K) throw TensorError("matmul: inner dimensions do not match");
    std::vector<int64_t> out_shape(as.begin(), as.end());
    out_shape.back() = N;
    auto out = make(out_shape);
    const int64_t lead = as.size() >= 2 ? prod(as, 0, as.size() - 2) : 1;
    if (bs.size() == 2 && detail::compute_bf16() && K % 8 == 0 && N % 8 == 0 && lead * M > 0) {
        // bf16 operands on the tensor cores, fp32 accumulation and result: A [T,K] x (B as [N,K])^T through mft_gemm_nt
        auto a_bf = detail::to_bf16(a);
        TensorPtr b_nk;
        if (trans_b) {
            b_nk = detail::to_bf16(b_in->dtype() == kBFloat16 ? b_in : b);
        } else {
            b_nk = std::make_shared<Tensor>(std::vector<int64_t>{N, K}, kBFloat16, kCPU);
            if (b_in->dtype() == kBFloat16) check(mft_transpose_bf16(b_in->device_read(), b_nk->device_write(), K, N, stream()), "matmul: operand transpose");
            else check(mft_transpose_f32_to_bf16((const float*)b->device_read(), b_nk->device_write(), K, N, stream()), "matmul: operand transpose");
        }
        check(mft_gemm_nt(a_bf->device_read(), K, b_nk->device_read(), K, lead * M, N, K, nullptr, 0, nullptr, 0, 0, nullptr, 1.0f,
                          out->device_write(), N, MFT_F32, 0, stream()), "matmul (tensor cores)");
        return out;
    }
    if (bs.size() == 2) {
        check(mft_matmul_f32((const float*)a->device_read(), (const float*)b->device_read(), (float*)out->device_write(), 1, lead * M, N, K, 0, 0, 0,
                             trans_b ? 1 : 0, stream()), "matmul");
    } else {
        if (prod(bs, 0, bs.size() - 2) != lead) throw TensorError("matmul: batch dimensions do not match");
        check(mft_matmul_f32((const float*)a->device_read(), (const float*)b->device_read(), (float*)out->device_write(), lead, M, N, K, M * K,
                             bs[bs.size() - 2] * bs.back(), M * N, trans_b ? 1 : 0, stream()), "matmul");
    }
    return out;
}

TensorPtr swap_last2(const TensorPtr& t) {
    std::vector<int> d(t->shape().size());
    std::iota(d.begin(), d.end(), 0);
    std::swap(d[d.size() - 1], d[d.size() - 2]);
    return permute_raw(t, d);
}

// dB for C = A x B: B 2-D shared -> (A flattened)^T x G ; batched -> A^T x G per batch.
TensorPtr grad_rhs(const TensorPtr& a, const TensorPtr& g, const std::vector<int64_t>& b_shape, bool b_is_transposed) {
    TensorPtr a2 = a, g2 = g;
    if (b_shape.size() == 2) {
        a2 = a->reshape({-1, a->shape().back()});
        g2 = g->reshape({-1, g->shape().back()});
    }
    // b [K,N]: dB = A^T G ; b [N,K] (rhs_T): dB = G^T A
    return b_is_transposed ? matmul_raw(swap_last2(g2), a2, false) : matmul_raw(swap_last2(a2), g2, false);
}

}  // namespace

void register_backward(const TensorPtr& out, const std::vector<TensorPtr>& inputs, BackwardFunctionPtr fn) {
    bool any = false;
    for (auto& t : inputs) any = any || (t && t->requires_grad());
    if (!any) return;
    out->set_requires_grad(true);
    autograd::Engine::instance().register_node(out, inputs, std::move(fn));
}

// ---------------------------------------------------------------- shapes
bool same_shape(const TensorPtr& a, const TensorPtr& b) { return a->shape() == b->shape(); }
std::vector<int64_t> infer_broadcast_shape(const TensorPtr& a, const TensorPtr& b) {
    const auto& x = a->shape();
    const auto& y = b->shape();
    const size_t n = std::max(x.size(), y.size());
    std::vector<int64_t> out(n);
    for (size_t i = 0; i < n; ++i) {
        const int64_t dx = i < n - x.size() ? 1 : x[i - (n - x.size())];
        const int64_t dy = i < n - y.size() ? 1 : y[i - (n - y.size())];
        if (dx != dy && dx != 1 && dy != 1) throw TensorError("shapes are not broadcastable");
        out[i] = std::max(dx, dy);
    }
    return out;
}
std::vector<int64_t> broadcast_shape(const TensorPtr& a, const TensorPtr& b) { return infer_broadcast_shape(a, b); }
bool broadcastable(const TensorPtr& a, const TensorPtr& b) {
    try { infer_broadcast_shape(a, b); return true; } catch (const TensorError&) { return false; }
}

// ---------------------------------------------------------------- arithmetic
TensorPtr add(const TensorPtr& a, const TensorPtr& b) {
    auto out = binary(MFT_EW_ADD, a, b);
    const auto sa = a->shape(), sb = b->shape();
    register_backward(out, {a, b}, closure([sa, sb](const TensorPtr& g) { return std::vector<TensorPtr>{sum_to_shape(g, sa), sum_to_shape(g, sb)}; }));
    return out;
}
TensorPtr sub(const TensorPtr& a, const TensorPtr& b) {
    auto out = binary(MFT_EW_SUB, a, b);
    const auto sa = a->shape(), sb = b->shape();
    register_backward(out, {a, b}, closure([sa, sb](const TensorPtr& g) {
        return std::vector<TensorPtr>{sum_to_shape(g, sa), sum_to_shape(unary(MFT_UN_NEG, g), sb)};
    }));
    return out;
}
TensorPtr mul(const TensorPtr& a, const TensorPtr& b) {
    auto out = binary(MFT_EW_MUL, a, b);
    register_backward(out, {a, b}, closure([a, b](const TensorPtr& g) {
        return std::vector<TensorPtr>{sum_to_shape(binary(MFT_EW_MUL, g, b), a->shape()), sum_to_shape(binary(MFT_EW_MUL, g, a), b->shape())};
    }));
    return out;
}
TensorPtr div(const TensorPtr& a, const TensorPtr& b) {
    auto out = binary(MFT_EW_DIV, a, b);
    register_backward(out, {a, b}, closure([a, b, out](const TensorPtr& g) {
        auto ga = binary(MFT_EW_DIV, g, b);
        auto gb = unary(MFT_UN_NEG, binary(MFT_EW_DIV, binary(MFT_EW_MUL, g, out), b));
        return std::vector<TensorPtr>{sum_to_shape(ga, a->shape()), sum_to_shape(gb, b->shape())};
    }));
    return out;
}
TensorPtr add(const TensorPtr& t, float s) {
    auto out = scalar_op(MFT_EW_ADD, t, s, false);
    register_backward(out, {t}, closure([](const TensorPtr& g) { return std::vector<TensorPtr>{g}; }));
    return out;
}
TensorPtr sub(const TensorPtr& t, float s) { return add(t, -s); }
TensorPtr mul(const TensorPtr& t, float s) {
    auto out = scalar_op(MFT_EW_MUL, t, s, false);
    register_backward(out, {t}, closure([s](const TensorPtr& g) { return std::vector<TensorPtr>{scalar_op(MFT_EW_MUL, g, s, false)}; }));
    return out;
}
TensorPtr div(const TensorPtr& t, float s) { return mul(t, 1.0f / s); }
TensorPtr add(float s, const TensorPtr& t) { return add(t, s); }
TensorPtr mul(float s, const TensorPtr& t) { return mul(t, s); }
TensorPtr sub(float s, const TensorPtr& t) {
    auto out = scalar_op(MFT_EW_SUB, t, s, true);
    register_backward(out, {t}, closure([](const TensorPtr& g) { return std::vector<TensorPtr>{unary(MFT_UN_NEG, g)}; }));
    return out;
}
TensorPtr div(float s, const TensorPtr& t) {
    auto out = scalar_op(MFT_EW_DIV, t, s, true);
    register_backward(out, {t}, closure([t, out](const TensorPtr& g) {
        return std::vector<TensorPtr>{unary(MFT_UN_NEG, binary(MFT_EW_DIV, binary(MFT_EW_MUL, g, out), t))};
    }));
    return out;
}

// ---------------------------------------------------------------- matmul family
TensorPtr matmul(const TensorPtr& a, const TensorPtr& b) {
    if (!a || !b) throw TensorError("matmul: null tensor");
    if (DTypeUtils::size_of(b->dtype()) == 2 && b->requires_grad()) throw TensorError("matmul: low-precision right operand must be frozen");
    const auto& bs = b->shape();
    // as the reference: a right operand stored [N,K] is used transposed when only that orientation fits
    const int64_t K = a->shape().back();
    const bool as_transposed = bs.size() == 2 && bs[0] != K && bs[1] == K;
    if (as_transposed) return matmul_rhs_T(a, b);
    auto out = matmul_raw(a, b, false);
    register_backward(out, {a, b}, closure([a, b](const TensorPtr& g) {
        std::vector<TensorPtr> r(2);
        if (a->requires_grad()) r[0] = matmul_raw(g, b, true);                                  // dA = G B^T
        if (b->requires_grad()) r[1] = grad_rhs(a, g, b->shape(), false);
        return r;
    }));
    return out;
}
TensorPtr matmul_rhs_T(const TensorPtr& a, const TensorPtr& b) {
    if (!a || !b) throw TensorError("matmul_rhs_T: null tensor");
    if (DTypeUtils::size_of(b->dtype()) == 2 && b->requires_grad()) throw TensorError("matmul_rhs_T: low-precision right operand must be frozen");
    auto out = matmul_raw(a, b, true);
    register_backward(out, {a, b}, closure([a, b](const TensorPtr& g) {
        std::vector<TensorPtr> r(2);
        if (a->requires_grad()) r[0] = matmul_raw(g, b, false);                                 // dA = G B
        if (b->requires_grad()) r[1] = grad_rhs(a, g, b->shape(), true);
        return r;
    }));
    return out;
}
TensorPtr linear(const TensorPtr& input, const TensorPtr& weight, const TensorPtr& bias) {
    auto y = matmul(input, weight);
    return bias ? add(y, bias) : y;
}

TensorPtr permute(const TensorPtr& t, const std::vector<int>& dims) {
    auto out = permute_raw(t, dims);
    const int nd = (int)dims.size();
    std::vector<int> inv((size_t)nd);
    for (int k = 0; k < nd; ++k) inv[(size_t)(dims[(size_t)k] < 0 ? dims[(size_t)k] + nd : dims[(size_t)k])] = k;
    register_backward(out, {t}, closure([inv](const TensorPtr& g) { return std::vector<TensorPtr>{permute_raw(g, inv)}; }));
    return out;
}
TensorPtr transpose(const TensorPtr& t, int d0, int d1) {
    const int nd = (int)t->shape().size();
    if (d0 < 0) d0 += nd;
    if (d1 < 0) d1 += nd;
    if (d0 < 0 || d1 < 0 || d0 >= nd || d1 >= nd) throw TensorError("transpose: dimension out of range");
    std::vector<int> d((size_t)nd);
    std::iota(d.begin(), d.end(), 0);
    std::swap(d[(size_t)d0], d[(size_t)d1]);
    return permute(t, d);
}

TensorPtr reshape(const TensorPtr& t, const std::vector<int64_t>& shape) {
    auto out = t->reshape(shape);
    out->set_requires_grad(false);
    const auto in_shape = t->shape();
    register_backward(out, {t}, closure([in_shape](const TensorPtr& g) { return std::vector<TensorPtr>{g->reshape(in_shape)}; }));
    return out;
}
TensorPtr view(const TensorPtr& t, const std::vector<int64_t>& shape) { return reshape(t, shape); }
TensorPtr flatten(const TensorPtr& t, int start, int end) {
    const int nd = (int)t->shape().size();
    if (start < 0) start += nd;
    if (end < 0) end += nd;
    std::vector<int64_t> s(t->shape().begin(), t->shape().begin() + start);
    s.push_back(prod(t->shape(), (size_t)start, (size_t)end + 1));
    s.insert(s.end(), t->shape().begin() + end + 1, t->shape().end());
    return reshape(t, s);
}
TensorPtr squeeze(const TensorPtr& t, int dim) { return reshape(t, t->squeeze(dim)->shape()); }
TensorPtr unsqueeze(const TensorPtr& t, int dim) { return reshape(t, t->unsqueeze(dim)->shape()); }

// ---------------------------------------------------------------- activations
TensorPtr gelu(const TensorPtr& x) {
    auto out = unary(MFT_UN_GELU, x);
    register_backward(out, {x}, closure([x](const TensorPtr& g) { return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, unary(MFT_UN_GELU_GRAD, x))}; }));
    return out;
}
TensorPtr relu(const TensorPtr& x) {
    auto out = unary(MFT_UN_RELU, x);
    register_backward(out, {x}, closure([x, out](const TensorPtr& g) {
        auto mask = binary(MFT_EW_DIV, out, scalar_op(MFT_EW_ADD, unary(MFT_UN_ABS, x), 1e-30f, false));   // 1 where x > 0, else 0
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, mask)};
    }));
    return out;
}
TensorPtr sigmoid(const TensorPtr& x) {
    auto out = unary(MFT_UN_SIGMOID, x);
    register_backward(out, {x}, closure([out](const TensorPtr& g) {
        auto d = binary(MFT_EW_MUL, out, scalar_op(MFT_EW_SUB, out, 1.0f, true));
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, d)};
    }));
    return out;
}
TensorPtr silu(const TensorPtr& x) {
    auto out = unary(MFT_UN_SILU, x);
    register_backward(out, {x}, closure([x](const TensorPtr& g) {
        auto s = unary(MFT_UN_SIGMOID, x);
        auto inner = scalar_op(MFT_EW_ADD, binary(MFT_EW_MUL, x, scalar_op(MFT_EW_SUB, s, 1.0f, true)), 1.0f, false);   // 1 + x (1 - s)
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, binary(MFT_EW_MUL, s, inner))};
    }));
    return out;
}
TensorPtr tanh_op(const TensorPtr& x) {
    auto out = unary(MFT_UN_TANH, x);
    register_backward(out, {x}, closure([out](const TensorPtr& g) {
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, scalar_op(MFT_EW_SUB, binary(MFT_EW_MUL, out, out), 1.0f, true))};
    }));
    return out;
}
TensorPtr exp(const TensorPtr& t) {
    auto out = unary(MFT_UN_EXP, t);
    register_backward(out, {t}, closure([out](const TensorPtr& g) { return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, out)}; }));
    return out;
}
TensorPtr log(const TensorPtr& t) {
    auto out = unary(MFT_UN_LOG, t);
    register_backward(out, {t}, closure([t](const TensorPtr& g) { return std::vector<TensorPtr>{binary(MFT_EW_DIV, g, t)}; }));
    return out;
}
TensorPtr sqrt(const TensorPtr& t) {
    auto out = unary(MFT_UN_SQRT, t);
    register_backward(out, {t}, closure([out](const TensorPtr& g) { return std::vector<TensorPtr>{binary(MFT_EW_DIV, scalar_op(MFT_EW_MUL, g, 0.5f, false), out)}; }));
    return out;
}
TensorPtr abs(const TensorPtr& t) {
    auto out = unary(MFT_UN_ABS, t);
    register_backward(out, {t}, closure([t, out](const TensorPtr& g) {
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, binary(MFT_EW_DIV, t, scalar_op(MFT_EW_ADD, out, 1e-30f, false)))};
    }));
    return out;
}
TensorPtr pow(const TensorPtr& t, float e) {
    auto out = unary(MFT_UN_POW, t, e);
    register_backward(out, {t}, closure([t, e](const TensorPtr& g) {
        return std::vector<TensorPtr>{binary(MFT_EW_MUL, g, scalar_op(MFT_EW_MUL, unary(MFT_UN_POW, t, e - 1.0f), e, false))};
    }));
    return out;
}
TensorPtr swiglu(const TensorPtr& gate, const TensorPtr& up) {
    require_f32(gate, "swiglu"); require_f32(up, "swiglu");
    if (!same_shape(gate, up)) throw std::runtime_error("gate and up tensors must have the same shape for SwiGLU");
    auto out = make(gate->shape());
    check(mft_swiglu_f32((const float*)gate->device_read(), (const float*)up->device_read(), nullptr, (float*)out->device_write(), nullptr, gate->numel(), stream()), "swiglu");
    register_backward(out, {gate, up}, closure([gate, up](const TensorPtr& g) {
        auto dg = make(gate->shape()), du = make(gate->shape());
        check(mft_swiglu_f32((const float*)gate->device_read(), (const float*)up->device_read(), (const float*)g->device_read(), (float*)dg->device_write(),
                             (float*)du->device_write(), gate->numel(), stream()), "swiglu backward");
        return std::vector<TensorPtr>{dg, du};
    }));
    return out;
}

// ---------------------------------------------------------------- softmax, reductions
TensorPtr softmax(const TensorPtr& x, int dim) {
    require_f32(x, "softmax");
    const int nd = (int)x->shape().size();
    if (dim < 0) dim += nd;
    if (dim != nd - 1) {      // move the softmax dimension last, apply, move back
        auto xt = transpose(x, dim, nd - 1);
        return transpose(softmax(xt, -1), dim, nd - 1);
    }
    const int64_t d = x->shape().back(), rows = x->numel() / d;
    auto out = make(x->shape());
    check(mft_softmax_f32((const float*)x->device_read(), (float*)out->device_write(), rows, d, stream()), "softmax");
    register_backward(out, {x}, closure([out, rows, d](const TensorPtr& g) {
        auto dx = make(out->shape());
        check(mft_softmax_bwd_f32((const float*)out->device_read(), (const float*)g->device_read(), (float*)dx->device_write(), rows, d, stream()), "softmax backward");
        return std::vector<TensorPtr>{dx};
    }));
    return out;
}
TensorPtr log_softmax(const TensorPtr& x, int dim) { return log(softmax(x, dim)); }

TensorPtr sum(const TensorPtr& t, int dim, bool keepdim) {
    require_f32(t, "sum");
    const auto shape = t->shape();
    const int nd = (int)shape.size();
    if (dim == -1) {     // the reference's convention: -1 reduces every element
        auto out = make({1});
        check(mft_reduce_sum_f32((const float*)t->device_read(), (float*)out->device_write(), 1, t->numel(), 1, 1.0f, stream()), "sum");
        register_backward(out, {t}, closure([shape](const TensorPtr& g) {
            auto full = make(shape);
            const std::vector<int64_t> one{1};
            check(mft_ew_binary_f32(MFT_EW_ADD, (const float*)full->device_read(), shape.data(), (int)shape.size(), (const float*)g->device_read(), one.data(), 1,
                                    (float*)full->device_readwrite(), shape.data(), (int)shape.size(), stream()), "sum backward");
            return std::vector<TensorPtr>{full};
        }));
        return out;
    }
    if (dim < 0) dim += nd;
    if (dim < 0 || dim >= nd) throw TensorError("sum: dimension out of range");
    std::vector<int64_t> rs, keep = shape;
    keep[(size_t)dim] = 1;
    for (int i = 0; i < nd; ++i) {
        if (i != dim) rs.push_back(shape[(size_t)i]);
        else if (keepdim) rs.push_back(1);
    }
    if (rs.empty()) rs.push_back(1);
    auto out = make(rs);
    const int64_t outer = prod(shape, 0, (size_t)dim), red = shape[(size_t)dim], inner = prod(shape, (size_t)dim + 1, shape.size());
    check(mft_reduce_sum_f32((const float*)t->device_read(), (float*)out->device_write(), outer, red, inner, 1.0f, stream()), "sum");
    register_backward(out, {t}, closure([shape, keep](const TensorPtr& g) {
        auto gk = g->reshape(keep);
        auto full = make(shape);
        check(mft_ew_binary_f32(MFT_EW_ADD, (const float*)full->device_read(), shape.data(), (int)shape.size(), (const float*)gk->device_read(), keep.data(),
                                (int)keep.size(), (float*)full->device_readwrite(), shape.data(), (int)shape.size(), stream()), "sum backward");
        return std::vector<TensorPtr>{full};
    }));
    return out;
}
TensorPtr mean(const TensorPtr& t, int dim, bool keepdim) {
    const float count = dim == -1 ? (float)t->numel() : (float)t->shape()[(size_t)(dim < 0 ? dim + (int)t->shape().size() : dim)];
    return mul(sum(t, dim, keepdim), 1.0f / count);
}

// ---------------------------------------------------------------- norms
static TensorPtr rms_norm_impl(const TensorPtr& x, const TensorPtr& w, float eps, int unit_offset, bool always_grad) {
    require_f32(x, "rms_norm"); require_f32(w, "rms_norm");
    const int64_t d = x->shape().back(), rows = x->numel() / d;
    if (w->numel() != d) throw TensorError("rms_norm: weight size mismatch");
    auto out = make(x->shape());
    auto rstd = make({rows});
    check(mft_rmsnorm_fwd(x->device_read(), MFT_F32, (const float*)w->device_read(), eps, unit_offset, out->device_write(), MFT_F32,
                          (float*)rstd->device_write(), nullptr, nullptr, rows, d, stream()), "rms_norm");
    auto fn = closure([x, w, rstd, eps, unit_offset, rows, d](const TensorPtr& g) {
        auto dx = make(x->shape());
        auto dw = make(w->shape());
        check(mft_rmsnorm_bwd(g->device_read(), MFT_F32, x->device_read(), MFT_F32, (const float*)w->device_read(), (const float*)rstd->device_read(), eps,
                              unit_offset, dx->device_write(), MFT_F32, 0, (float*)dw->device_readwrite(), rows, d, stream()), "rms_norm backward");
        return std::vector<TensorPtr>{dx, dw};
    });
    if (always_grad) {   // the reference's rms_norm marks its output as requiring grad unconditionally
        out->set_requires_grad(true);
        autograd::Engine::instance().register_node(out, {x, w}, fn);
    } else {
        register_backward(out, {x, w}, fn);
    }
    return out;
}
TensorPtr rms_norm(const TensorPtr& x, const TensorPtr& w, float eps) { return rms_norm_impl(x, w, eps, 1, true); }
TensorPtr rms_norm_affine(const TensorPtr& x, const TensorPtr& w, float eps) { return rms_norm_impl(x, w, eps, 0, false); }

TensorPtr layer_norm(const TensorPtr& x, const TensorPtr& w, const TensorPtr& b, float eps) {
    require_f32(x, "layer_norm"); require_f32(w, "layer_norm"); require_f32(b, "layer_norm");
    const int64_t d = x->shape().back(), rows = x->numel() / d;
    auto out = make(x->shape());
    auto mean_t = make({rows}), rstd = make({rows});
    check(mft_layernorm_fwd(x->device_read(), MFT_F32, (const float*)w->device_read(), (const float*)b->device_read(), eps, out->device_write(), MFT_F32,
                            (float*)mean_t->device_write(), (float*)rstd->device_write(), rows, d, stream()), "layer_norm");
    register_backward(out, {x, w, b}, closure([x, w, mean_t, rstd, rows, d](const TensorPtr& g) {
        auto dx = make(x->shape());
        auto dw = make(w->shape()), db = make(w->shape());
        check(mft_layernorm_bwd(g->device_read(), MFT_F32, x->device_read(), MFT_F32, (const float*)w->device_read(), (const float*)mean_t->device_read(),
                                (const float*)rstd->device_read(), dx->device_write(), MFT_F32, 0, (float*)dw->device_readwrite(),
                                (float*)db->device_readwrite(), rows, d, stream()), "layer_norm backward");
        return std::vector<TensorPtr>{dx, dw, db};
    }));
    return out;
}

// ---------------------------------------------------------------- attention helpers
TensorPtr create_causal_mask(int seq_len, DType dtype, Device device) {
    if (dtype != kFloat32) throw TensorError("create_causal_mask: float32 only");
    auto m = std::make_shared<Tensor>(std::vector<int64_t>{seq_len, seq_len}, kFloat32, device);
    float* p = m->data<float>();
    for (int i = 0; i < seq_len; ++i)
        for (int j = i + 1; j < seq_len; ++j) p[(size_t)i * seq_len + j] = -1e10f;
    return m;
}

TensorPtr repeat_kv_heads(const TensorPtr& kv, int rep) {
    require_f32(kv, "repeat_kv_heads");
    if (kv->shape().size() != 4) throw TensorError("repeat_kv_heads: expected [batch, kv_heads, seq, head_dim]");
    if (rep == 1) return kv;
    const auto& s = kv->shape();
    auto out = make({s[0], s[1] * rep, s[2], s[3]});
    check(mft_repeat_kv(kv->device_read(), MFT_F32, out->device_write(), s[0], s[1], s[2], s[3], rep, stream()), "repeat_kv_heads");
    const auto shape = s;
    register_backward(out, {kv}, closure([shape, rep](const TensorPtr& g) {
        auto dkv = make(shape);
        check(mft_repeat_kv_bwd((const float*)g->device_read(), (float*)dkv->device_write(), shape[0], shape[1], shape[2], shape[3], rep, stream()), "repeat_kv backward");
        return std::vector<TensorPtr>{dkv};
    }));
    return out;
}

TensorPtr apply_rope(const TensorPtr& x, int seq_len, int head_dim, float theta) {
    require_f32(x, "apply_rope");
    const auto& s = x->shape();
    if (s.size() != 4) throw std::runtime_error("apply_rope expects 4D tensor [batch, heads, seq_len, head_dim]");
    if (s[2] != seq_len || s[3] != head_dim) throw std::runtime_error("apply_rope: seq_len/head_dim do not match the tensor");
    const int64_t half = head_dim / 2;
    auto cs = make({seq_len, half}), sn = make({seq_len, half});
    check(mft_rope_table_host(cs->data<float>(), sn->data<float>(), seq_len, head_dim, theta), "rope table");
    auto out = make(s);
    const int64_t rows = s[0] * s[1];
    check(mft_rope_f32((const float*)x->device_read(), (float*)out->device_write(), (const float*)cs->device_read(), (const float*)sn->device_read(), rows,
                       seq_len, head_dim, 0, stream()), "apply_rope");
    register_backward(out, {x}, closure([cs, sn, rows, seq_len, head_dim](const TensorPtr& g) {
        auto dx = make(g->shape());
        check(mft_rope_f32((const float*)g->device_read(), (float*)dx->device_write(), (const float*)cs->device_read(), (const float*)sn->device_read(), rows,
                           seq_len, head_dim, 1, stream()), "apply_rope backward");
        return std::vector<TensorPtr>{dx};
    }));
    return out;
}

// ---------------------------------------------------------------- slice (host side: index arithmetic, not on the step's path)
TensorPtr Tensor::slice(int dim, int64_t start, int64_t end, int64_t step) const {
    const int nd = (int)shape_.size();
    if (dim < 0) dim += nd;
    if (dim < 0 || dim >= nd) throw TensorError("slice: dimension out of range");
    if (step <= 0) throw TensorError("slice: step must be positive");
    const int64_t len = shape_[(size_t)dim];
    if (start < 0) start += len;
    if (end < 0) end += len;
    start = std::max<int64_t>(0, std::min(start, len));
    end = std::max<int64_t>(start, std::min(end, len));
    const int64_t n_out = (end - start + step - 1) / step;
    std::vector<int64_t> os = shape_;
    os[(size_t)dim] = n_out;
    auto out = std::make_shared<Tensor>(os, dtype_, device_);
    const size_t es = DTypeUtils::size_of(dtype_);
    const int64_t outer = prod(shape_, 0, (size_t)dim), inner = prod(shape_, (size_t)dim + 1, shape_.size());
    const char* src = static_cast<const char*>(data_ptr());
    char* dst = static_cast<char*>(out->data_ptr());
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t k = 0; k < n_out; ++k)
            std::memcpy(dst + ((o * n_out + k) * inner) * es, src + ((o * len + start + k * step) * inner) * es, (size_t)inner * es);
    if (dtype_ == kFloat32) {
        const auto in_shape = shape_;
        register_backward(out, {self()}, closure([in_shape, dim, start, step, n_out, outer, inner, len](const TensorPtr& g) {
            auto dx = std::make_shared<Tensor>(in_shape, kFloat32, kCPU);
            const float* gs = g->data<float>();
            float* d = dx->data<float>();
            for (int64_t o = 0; o < outer; ++o)
                for (int64_t k = 0; k < n_out; ++k)
                    for (int64_t i = 0; i < inner; ++i) d[(o * len + start + k * step) * inner + i] += gs[(o * n_out + k) * inner + i];
            (void)dim;
            return std::vector<TensorPtr>{dx};
        }));
    }
    return out;
}

}  // namespace ops
