// Operator surface of the API (namespace ops), same names and argument meaning
// as the reference's core/ops.h.  Every function runs on the GPU through the C
// ABI of libmft_cuda.so and records an autograd node when an input requires grad.
//
// Arithmetic type.  By default the eager operators compute in fp32 (generic
// kernels): that is what the reference's unit tests, with their 1e-5 bounds,
// expect.  With the compute type set to bf16 (set_compute_dtype(kBFloat16), or
// MFT_COMPUTE_DTYPE=bf16 in the environment) the operators that have a fused
// tensor-core kernel use it: matmul / matmul_rhs_T / linear with a 2-D right
// operand (and so LoRALinear::forward) run mft_gemm_nt, memory_efficient_attention
// runs mft_attn_fwd / mft_attn_bwd, selected_token / streaming_lm_cross_entropy
// run mft_lmhead_ce_fwd / _bwd; inputs are rounded to bf16, products accumulate
// in fp32, results come back as fp32 tensors.  The models' own forward() always
// runs the bf16 step engine, whatever this switch says.
#pragma once
#include <string>
#include <vector>

#include "backward_functions.h"
#include "tensor.h"

namespace ops {

TensorPtr add(const TensorPtr& a, const TensorPtr& b);
TensorPtr sub(const TensorPtr& a, const TensorPtr& b);
TensorPtr mul(const TensorPtr& a, const TensorPtr& b);
TensorPtr div(const TensorPtr& a, const TensorPtr& b);
TensorPtr add(const TensorPtr& t, float s);
TensorPtr sub(const TensorPtr& t, float s);
TensorPtr mul(const TensorPtr& t, float s);
TensorPtr div(const TensorPtr& t, float s);
TensorPtr add(float s, const TensorPtr& t);
TensorPtr sub(float s, const TensorPtr& t);
TensorPtr mul(float s, const TensorPtr& t);
TensorPtr div(float s, const TensorPtr& t);

TensorPtr matmul(const TensorPtr& a, const TensorPtr& b);          // a [..,M,K] x b [K,N] or [..,K,N]
TensorPtr matmul_rhs_T(const TensorPtr& a, const TensorPtr& b);    // a [..,M,K] x b [N,K]^T
TensorPtr transpose(const TensorPtr& t, int dim0, int dim1);
TensorPtr permute(const TensorPtr& t, const std::vector<int>& dims);
TensorPtr linear(const TensorPtr& input, const TensorPtr& weight, const TensorPtr& bias = nullptr);

TensorPtr relu(const TensorPtr& x);
TensorPtr gelu(const TensorPtr& x);
TensorPtr silu(const TensorPtr& x);
TensorPtr sigmoid(const TensorPtr& x);
TensorPtr tanh_op(const TensorPtr& x);
inline TensorPtr tanh(const TensorPtr& x) { return tanh_op(x); }
TensorPtr softmax(const TensorPtr& x, int dim = -1);
TensorPtr log_softmax(const TensorPtr& x, int dim = -1);

TensorPtr layer_norm(const TensorPtr& input, const TensorPtr& weight, const TensorPtr& bias, float eps = 1e-5f);
TensorPtr rms_norm(const TensorPtr& input, const TensorPtr& weight, float eps = 1e-6f);          // scale (1 + w)
TensorPtr rms_norm_affine(const TensorPtr& input, const TensorPtr& weight, float eps = 1e-6f);   // scale w

TensorPtr reshape(const TensorPtr& t, const std::vector<int64_t>& shape);
TensorPtr view(const TensorPtr& t, const std::vector<int64_t>& shape);
TensorPtr cast(const TensorPtr& t, DType target);
inline TensorPtr to_fp16(const TensorPtr& t) { return cast(t, DType::kFloat16); }
inline TensorPtr to_fp32(const TensorPtr& t) { return cast(t, DType::kFloat32); }
TensorPtr flatten(const TensorPtr& t, int start_dim = 0, int end_dim = -1);
TensorPtr squeeze(const TensorPtr& t, int dim = -1);
TensorPtr unsqueeze(const TensorPtr& t, int dim);

TensorPtr sum(const TensorPtr& t, int dim = -1, bool keepdim = false);    // dim == -1 reduces everything to shape {1}
TensorPtr mean(const TensorPtr& t, int dim = -1, bool keepdim = false);

TensorPtr abs(const TensorPtr& t);
TensorPtr sqrt(const TensorPtr& t);
TensorPtr exp(const TensorPtr& t);
TensorPtr log(const TensorPtr& t);
TensorPtr pow(const TensorPtr& t, float exponent);

TensorPtr create_causal_mask(int seq_len, DType dtype = kFloat32, Device device = kCPU);   // 0 on/below the diagonal, -1e10 above
TensorPtr repeat_kv_heads(const TensorPtr& kv, int repeat_factor);
TensorPtr apply_rope(const TensorPtr& x, int seq_len, int head_dim, float rope_theta = 10000.0f);
TensorPtr swiglu(const TensorPtr& gate, const TensorPtr& up);

bool same_shape(const TensorPtr& a, const TensorPtr& b);
bool broadcastable(const TensorPtr& a, const TensorPtr& b);
std::vector<int64_t> broadcast_shape(const TensorPtr& a, const TensorPtr& b);
std::vector<int64_t> infer_broadcast_shape(const TensorPtr& a, const TensorPtr& b);

// kFloat32 (default) or kBFloat16: see the head of this file.
void set_compute_dtype(DType dtype);
DType compute_dtype();

// Registers `fn` as the backward rule of `out` if any input requires grad.
void register_backward(const TensorPtr& out, const std::vector<TensorPtr>& inputs, BackwardFunctionPtr fn);

}  // namespace ops

