#include "lora_linear.h"

#include <cstring>
#include <stdexcept>

#include "../core/autograd_engine.h"
#include "../core/ops.h"

namespace ops {

namespace {
// A is [in,r] (GPT-2 / Qwen injectors) or [r,in] (PEFT layout); return it as [in,r].
TensorPtr a_in_r(const TensorPtr& A, int64_t in) {
    if (A->shape().size() != 2) throw std::runtime_error("LoRALinear: A must be 2-D");
    if (A->shape()[0] == in) return A;
    if (A->shape()[1] == in) return transpose(A, 0, 1);
    throw std::runtime_error("LoRALinear: A does not match the layer's input width");
}
// B is [r,cols] or [cols,r]; return it as [r,cols].
TensorPtr b_r_cols(const TensorPtr& B, int64_t r, int64_t cols) {
    if (B->shape().size() != 2) throw std::runtime_error("LoRALinear: B must be 2-D");
    if (B->shape()[0] == r && B->shape()[1] == cols) return B;
    if (B->shape()[1] == r && B->shape()[0] == cols) return transpose(B, 0, 1);
    throw std::runtime_error("LoRALinear: B does not match rank / column count");
}
}  // namespace

void LoRALinear::attach_lora(const TensorPtr& A, const TensorPtr& B, float scale, int col0, int cols) {
    if (!A || !B) throw std::runtime_error("LoRALinear::attach_lora: null tensor");
    if (merged_) throw std::runtime_error("LoRALinear::attach_lora: unmerge before attaching");
    const int64_t out = W_->shape()[1];
    if (cols < 0) cols = (int)out - col0;
    if (col0 < 0 || col0 + cols > out) throw std::runtime_error("LoRALinear::attach_lora: column range outside the base weight");
    slices_.emplace_back(A, B, scale, col0, cols);
}

void LoRALinear::clear_lora() {
    if (merged_) unmerge_from_base();
    slices_.clear();
}

std::vector<TensorPtr> LoRALinear::trainable_parameters() const {
    std::vector<TensorPtr> p;
    for (const auto& s : slices_) { p.push_back(s.A); p.push_back(s.B); }
    return p;
}

std::vector<std::pair<std::string, TensorPtr>> LoRALinear::debug_params() const {
    std::vector<std::pair<std::string, TensorPtr>> p;
    for (size_t i = 0; i < slices_.size(); ++i) {
        const std::string base = debug_name_ + ".slice" + std::to_string(i);
        p.emplace_back(base + ".A", slices_[i].A);
        p.emplace_back(base + ".B", slices_[i].B);
    }
    return p;
}

void LoRALinear::merge_to_base() {
    if (merged_ || slices_.empty()) return;
    autograd::NoGradGuard ng;
    const int64_t in = W_->shape()[0], out = W_->shape()[1];
    merge_backup_.assign(static_cast<const uint8_t*>(static_cast<const Tensor&>(*W_).data_ptr()),
                         static_cast<const uint8_t*>(static_cast<const Tensor&>(*W_).data_ptr()) + W_->nbytes());
    for (const auto& s : slices_) {
        auto A = a_in_r(s.A, in);
        auto B = b_r_cols(s.B, A->shape()[1], s.cols);
        auto delta = mul(matmul(A, B), s.scale);            // [in, cols] on the GPU
        const float* d = static_cast<const Tensor&>(*delta).data<float>();
        if (W_->dtype() == kFloat32) {
            float* w = W_->data<float>();
            for (int64_t i = 0; i < in; ++i)
                for (int64_t j = 0; j < s.cols; ++j) w[i * out + s.col0 + j] += d[i * s.cols + j];
        } else if (W_->dtype() == kBFloat16 || W_->dtype() == kFloat16) {
            uint16_t* w = W_->data<uint16_t>();
            const bool bf = W_->dtype() == kBFloat16;
            for (int64_t i = 0; i < in; ++i)
                for (int64_t j = 0; j < s.cols; ++j) {
                    uint16_t& e = w[i * out + s.col0 + j];
                    const float v = (bf ? bf16_bits_to_float32(e) : fp16_bits_to_float32(e)) + d[i * s.cols + j];
                    e = bf ? float32_to_bf16_bits(v) : float32_to_fp16_bits(v);
                }
        } else {
            throw std::runtime_error("LoRALinear::merge_to_base: unsupported base dtype");
        }
    }
    merged_ = true;
}

void LoRALinear::unmerge_from_base() {
    if (!merged_) return;
    if (merge_backup_.size() != W_->nbytes()) throw std::runtime_error("LoRALinear::unmerge_from_base: missing backup");
    std::memcpy(W_->data_ptr(), merge_backup_.data(), merge_backup_.size());   // exact bytes, no arithmetic
    merge_backup_.clear();
    merged_ = false;
}

TensorPtr LoRALinear::forward(const TensorPtr& x) const {
    if (!x || x->shape().size() != 3) throw std::runtime_error("LoRALinear::forward expects x of shape [B, S, in]");
    const int64_t in = W_->shape()[0], out = W_->shape()[1];
    if (x->shape()[2] != in) throw std::runtime_error("LoRALinear::forward: input width does not match the base weight");
    TensorPtr y = matmul(x, W_);
    if (b_) y = add(y, b_);
    if (merged_) return y;
    for (const auto& s : slices_) {
        auto A = a_in_r(s.A, in);
        auto B = b_r_cols(s.B, A->shape()[1], s.cols);
        if (s.col0 == 0 && s.cols == out) {
            y = add(y, mul(matmul(matmul(x, A), B), s.scale));
        } else {
            // A slice that covers part of the columns only contributes to the forward value: the reference adds it
            // in place without recording it, so its A/B receive no gradient.  Same here.
            autograd::NoGradGuard ng;
            auto Bfull = std::make_shared<Tensor>(std::vector<int64_t>{B->shape()[0], out}, kFloat32, kCPU);
            const float* bsrc = static_cast<const Tensor&>(*B).data<float>();
            float* bdst = Bfull->data<float>();
            for (int64_t r = 0; r < B->shape()[0]; ++r)
                for (int64_t j = 0; j < s.cols; ++j) bdst[r * out + s.col0 + j] = bsrc[r * s.cols + j];
            auto delta = mul(matmul(matmul(x->detach(), A->detach()), Bfull), s.scale);
            const bool rg = y->requires_grad();
            auto y2 = add(y->detach(), delta);
            if (rg) {
                // keep y's own history: y2 = y + const
                autograd::Engine::instance().set_enabled(true);
                y = add(y, delta);
                autograd::Engine::instance().set_enabled(false);
            } else {
                y = y2;
            }
        }
    }
    return y;
}

}  // namespace ops
