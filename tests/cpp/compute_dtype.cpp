// The eager operators under both compute types: every case runs once in fp32 (generic kernels) and once with
// ops::set_compute_dtype(kBFloat16) (tensor-core GEMM, fused attention, fused lm head + loss) on the same inputs, and
// the bf16 results - values and gradients - must agree with the fp32 ones to bf16 rounding.
// Prints one line per case: name, cosine and largest error relative to the fp32 result's largest magnitude.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "core/lm_loss.h"
#include "core/memory_efficient_attention.h"
#include "core/ops.h"
#include "nn/lora_linear.h"

using namespace ops;

static std::mt19937 rng(1234);
static TensorPtr randn(const std::vector<int64_t>& shape, float std_dev, bool grad) {
    auto t = std::make_shared<Tensor>(shape, kFloat32, kCPU);
    std::normal_distribution<float> d(0.f, std_dev);
    float* p = t->data<float>();
    for (int64_t i = 0; i < t->numel(); ++i) p[i] = d(rng);
    t->set_requires_grad(grad);
    return t;
}
static std::vector<float> values(const TensorPtr& t) {
    const float* p = static_cast<const Tensor&>(*t).data<float>();
    return std::vector<float>(p, p + t->numel());
}
static int failures = 0;
static void compare(const std::string& name, const std::vector<float>& ref, const std::vector<float>& got, double min_cos, double max_rel) {
    double dot = 0, na = 0, nb = 0, amax = 0, emax = 0;
    if (ref.size() != got.size()) { std::printf("%-34s SIZE MISMATCH\n", name.c_str()); ++failures; return; }
    for (size_t i = 0; i < ref.size(); ++i) {
        dot += (double)ref[i] * got[i]; na += (double)ref[i] * ref[i]; nb += (double)got[i] * got[i];
        amax = std::max(amax, (double)std::fabs(ref[i])); emax = std::max(emax, (double)std::fabs(ref[i] - got[i]));
    }
    const double cos = dot / (std::sqrt(na) * std::sqrt(nb) + 1e-30), rel = emax / (amax + 1e-30);
    const bool ok = cos >= min_cos && rel <= max_rel && std::isfinite(cos);
    std::printf("%-34s cos %.6f  max err / max |ref| %.4f  %s\n", name.c_str(), cos, rel, ok ? "ok" : "FAIL");
    if (!ok) ++failures;
}

// runs `fn` (which returns the output and fills the leaf list) under both compute types
struct Run { std::vector<float> out; std::vector<std::vector<float>> grads; };
static Run run(DType dt, const std::function<TensorPtr()>& fn, const std::vector<TensorPtr>& leaves, const TensorPtr& weight) {
    set_compute_dtype(dt);
    for (auto& l : leaves) l->zero_grad();
    auto out = fn();
    TensorPtr loss = out->numel() == 1 ? out : sum(mul(out, weight));
    loss->backward();
    Run r;
    r.out = values(out);
    for (auto& l : leaves) r.grads.push_back(l->grad() ? values(l->grad()) : std::vector<float>());
    set_compute_dtype(kFloat32);
    return r;
}
static void both(const std::string& name, const std::function<TensorPtr()>& fn, const std::vector<TensorPtr>& leaves, const TensorPtr& weight,
                 double min_cos = 0.999, double max_rel = 2e-2) {
    Run a = run(kFloat32, fn, leaves, weight), b = run(kBFloat16, fn, leaves, weight);
    compare(name + " value", a.out, b.out, min_cos, max_rel);
    for (size_t i = 0; i < leaves.size(); ++i) compare(name + " grad " + std::to_string(i), a.grads[i], b.grads[i], min_cos, max_rel);
}

int main() {
    {   // matmul with a shared 2-D right operand, both orientations
        auto a = randn({3, 40, 64}, 1.f, true), b = randn({64, 48}, 0.3f, true), bt = randn({48, 64}, 0.3f, true);
        auto w = randn({3, 40, 48}, 1.f, false);
        both("matmul [3,40,64]x[64,48]", [&] { return matmul(a, b); }, {a, b}, w);
        both("matmul_rhs_T [3,40,64]x[48,64]^T", [&] { return matmul_rhs_T(a, bt); }, {a, bt}, w);
    }
    {   // LoRA linear: frozen base + bias, trainable A / B
        auto W = randn({64, 96}, 0.2f, false), bias = randn({96}, 0.1f, false);
        auto A = randn({64, 8}, 0.2f, true), B = randn({8, 96}, 0.2f, true);
        auto x = randn({2, 24, 64}, 1.f, true), w = randn({2, 24, 96}, 1.f, false);
        LoRALinear lin(W, bias);
        lin.attach_lora(A, B, 2.0f);
        both("LoRALinear [2,24,64]->96 r8", [&] { return lin.forward(x); }, {x, A, B}, w);
    }
    {   // causal attention, the mask implied and given
        auto q = randn({2, 4, 192, 64}, 1.f, true), k = randn({2, 4, 192, 64}, 1.f, true), v = randn({2, 4, 192, 64}, 1.f, true);
        auto w = randn({2, 4, 192, 64}, 1.f, false);
        both("memory_efficient_attention", [&] { return memory_efficient_attention(q, k, v); }, {q, k, v}, w);
        auto mask = create_causal_mask(192);
        both("memory_efficient_attention(mask)", [&] { return memory_efficient_attention(q, k, v, mask); }, {q, k, v}, w);
    }
    {   // lm head + shifted cross-entropy without the logits tensor
        auto h = randn({2, 24, 64}, 1.f, true), W = randn({1000, 64}, 0.2f, false);
        auto labels = std::make_shared<Tensor>(std::vector<int64_t>{2, 24}, kInt32, kCPU);
        std::uniform_int_distribution<int> d(0, 999);
        for (int i = 0; i < 48; ++i) labels->data<int32_t>()[i] = (i % 7 == 3) ? -100 : d(rng);
        both("streaming_lm_cross_entropy mean", [&] { return streaming_lm_cross_entropy(h, W, labels, -100, "mean"); }, {h}, nullptr);
        both("selected_token_lm_ce sum", [&] { return selected_token_lm_cross_entropy(h, W, labels, -100, "sum"); }, {h}, nullptr);
    }
    if (compute_dtype() != kFloat32) { std::printf("compute type was not restored\n"); ++failures; }
    std::printf(failures ? "FAILED %d\n" : "ALL OK\n", failures);
    return failures ? 1 : 0;
}
