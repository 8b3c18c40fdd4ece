// LoRA-augmented linear layer (same class and methods as the reference's nn/lora_linear.h):
//   y = x W (+ b) + sum_i scale_i * (x A_i) B_i          W [in,out], A_i [in,r], B_i [r,cols_i]
// Only A/B are trainable; W and b are frozen references to the base weights.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "../core/tensor.h"

namespace ops {

struct LoRASlice {
    TensorPtr A;
    TensorPtr B;
    float scale;   // alpha / rank
    int col0;      // first output column the slice adds to
    int cols;      // number of columns (-1: all)
    LoRASlice(const TensorPtr& a, const TensorPtr& b, float s, int c0 = 0, int c = -1) : A(a), B(b), scale(s), col0(c0), cols(c) {}
};

class LoRALinear {
public:
    LoRALinear(const TensorPtr& W_base, const TensorPtr& b_base = nullptr) : W_(W_base), b_(b_base), merged_(false) {}

    void attach_lora(const TensorPtr& A, const TensorPtr& B, float scale, int col0 = 0, int cols = -1);
    void clear_lora();                 // un-merges first if needed
    void merge_to_base();              // W[:, col0:col0+cols] += scale * A B   (inference / export)
    void unmerge_from_base();          // restores the exact pre-merge bytes
    TensorPtr forward(const TensorPtr& x) const;   // x [B,S,in] -> [B,S,out]

    void set_debug_name(const std::string& name) { debug_name_ = name; }
    std::vector<std::pair<std::string, TensorPtr>> debug_params() const;
    std::vector<TensorPtr> trainable_parameters() const;   // A then B per slice

    const TensorPtr& W() const { return W_; }
    const TensorPtr& b() const { return b_; }
    const std::vector<LoRASlice>& slices() const { return slices_; }
    bool is_merged() const { return merged_; }

private:
    TensorPtr W_;
    TensorPtr b_;
    std::vector<LoRASlice> slices_;
    bool merged_;
    std::vector<uint8_t> merge_backup_;
    std::string debug_name_;
};

}  // namespace ops
