// Step engine internals: the device-side counterpart of the reference's model
// graphs (GPT-2, Qwen2.5, Gemma-3 with LoRA) as a static schedule of kernels
// from mft_cuda.h over preallocated activations.
#pragma once
#include <cuda_bf16.h>

#include <string>
#include <vector>

#include "../../include/mft_step.h"

namespace mft {

typedef __nv_bfloat16 bf16;

// One frozen linear of the reference ([in, out] fp32 on the host).
struct LinearSlot {
    int in = 0, out = 0;
    int col0 = 0;             // first output column inside its fused group
    bool has_lora = false;
    int lora_idx = -1;        // index of A in the lora tensor list (B = +1)
    int panel_col = 0;        // first of its `rank` columns in the group's 64-wide LoRA panels
};

// Linears that share their input, executed as ONE GEMM: concatenated frozen
// weights in both K-major layouts plus the 64-wide LoRA panels.
struct LinearGroup {
    int in = 0, n_total = 0;
    std::vector<LinearSlot> slots;
    bf16* w_nk = nullptr;     // [n_total, in]   forward operand
    bf16* w_kn = nullptr;     // [in, n_total]   backward operand
    float* bias = nullptr;    // [n_total] or null
    bool any_lora = false;
    int k2 = 0;               // used panel columns
    bf16 *a_nk = nullptr, *a_kn = nullptr, *b_nk = nullptr, *b_kn = nullptr;   // [64,in] [in,64] [n_total,64] [64,n_total]
    float *da_pan = nullptr, *db_pan = nullptr;                                 // [in,64] [64,n_total] fp32 scratch
};

struct ParamInfo {
    std::string name;
    int64_t rows = 0, cols = 0;
    // where it goes on upload
    enum Kind { EMBED, POS_EMBED, LM_HEAD_COPY, NORM, LINEAR, BIAS } kind = NORM;
    float* f32_dst = nullptr;          // NORM / BIAS
    LinearGroup* group = nullptr;      // LINEAR / BIAS
    int slot = 0;
};

struct LoraInfo {
    int64_t rows = 0, cols = 0;
    int64_t offset = 0;       // into the flat buckets
    bool has_grad = true;
};

struct LayerBuffers {
    float* x = nullptr;        // [T,H] residual stream entering the layer (f32)
    bf16* h1 = nullptr;        // norm1 output
    float* rstd1 = nullptr; float* mean1 = nullptr;
    bf16* qkv = nullptr;       // [T, (nh+2nkv)*hd]
    bf16* xa_qkv = nullptr;    // [T,64]
    bf16* qk_r = nullptr;      // [T, (nh+nkv)*hd] after per-head norm + RoPE
    float *rstd_q = nullptr, *rstd_k = nullptr;
    bf16* o = nullptr;         // [T, nh*hd]
    float* lse = nullptr;
    bf16* xa_o = nullptr;
    bf16* attn_out = nullptr;  // [T,H]
    float* rstd2 = nullptr;
    float* x_mid = nullptr;    // [T,H]
    bf16* h2 = nullptr;
    float* rstd3 = nullptr; float* mean3 = nullptr;
    bf16* gu = nullptr;        // [T, 2I] (gate | up) or [T, I] for GPT-2
    bf16* xa_gu = nullptr;
    bf16* act = nullptr;       // [T, I]
    bf16* xa_d = nullptr;
    bf16* mlp_out = nullptr;   // [T,H]
    float* rstd4 = nullptr;
};

struct LayerWeights {
    float *ln1_w = nullptr, *ln1_b = nullptr, *ln2_w = nullptr, *ln2_b = nullptr;   // GPT-2 LN / Qwen+Gemma input & pre-ffn norms
    float *post_attn_w = nullptr, *post_ffn_w = nullptr;                           // Gemma
    float *q_norm_w = nullptr, *k_norm_w = nullptr;                                // Gemma
    LinearGroup qkv, o, gu, down;
    bool sliding = false;
};

}  // namespace mft

namespace mft {
bool gemm_profiling_enabled();   // per-launch GEMM event timing is on (it records events: incompatible with capture)
}

// One captured forward + backward (a fixed sequence of ~1100 launches for a given batch shape).
struct StepGraph {
    int64_t batch = 0, seq = 0, n_valid_global = 0;
    float loss_scale = 1.0f;
    int calls = 0;                   // eager runs seen with this key (the first one also performs one-time set-up)
    int64_t kernels = 0;             // kernel launches the graph holds (added to the library's launch counter per replay)
    cudaGraphExec_t exec = nullptr;
};

struct mft_model {
    mft_model_config_t cfg;
    cudaStream_t stream = nullptr;
    // Replay of the training step as a CUDA graph: the launches of one step are issued faster than the host can
    // make them one by one (tensor-map encodes + ~1100 launches per step).  Captured on a private stream that is
    // ordered against `stream` with events.  MFT_STEP_GRAPH=0 disables it.
    // double-buffered input: two device slots filled on a copy stream
    cudaStream_t copy_stream = nullptr;
    int32_t* slot_ids[2] = {nullptr, nullptr};
    int32_t* slot_labels[2] = {nullptr, nullptr};
    cudaEvent_t slot_ready[2] = {nullptr, nullptr}, slot_free[2] = {nullptr, nullptr};
    float loss_scale = 1.0f;         // d(loss) of the next backward passes (1 / grad_accum_steps under a step driver)
    bool use_graph = true;
    cudaStream_t graph_stream = nullptr;
    cudaEvent_t graph_in = nullptr, graph_out = nullptr;
    std::vector<StepGraph> graphs;
    int64_t max_tokens = 0;
    std::vector<void*> allocations;
    int64_t activation_bytes = 0;

    mft::bf16* embed = nullptr;      // [V,H]
    mft::bf16* embed_t = nullptr;    // [H, ld_t]
    int64_t ld_t = 0;
    mft::bf16* pos_embed = nullptr;  // GPT-2 [n_pos, H]
    float *final_w = nullptr, *final_b = nullptr;
    std::vector<mft::LayerWeights> layers;
    std::vector<mft::LayerBuffers> bufs;
    std::vector<mft::ParamInfo> params;
    std::vector<mft::LoraInfo> loras;

    // flat LoRA buckets
    float *p_bucket = nullptr, *g_bucket = nullptr, *m_bucket = nullptr, *v_bucket = nullptr;
    int64_t bucket_n = 0;
    int64_t adam_step = 0;
    float* sqnorm = nullptr;

    // pack / unpack tables (device)
    mft_block_copy_t *pack_table = nullptr, *unpack_table = nullptr;
    int n_pack = 0, n_unpack = 0;
    float* grad_pan_base = nullptr; int64_t grad_pan_floats = 0;
    bool panels_dirty = true;
    // LoRA merged into the frozen weights (evaluation / export): forward passes skip the adapter products, training
    // calls are refused.  The backups restore the weights byte for byte on unmerge.
    bool merged = false;
    struct MergeBackup { mft::LinearGroup* group; mft::bf16* w_nk; mft::bf16* w_kn; };
    std::vector<MergeBackup> merge_backup;

    // rope tables
    float *cos_g = nullptr, *sin_g = nullptr, *cos_l = nullptr, *sin_l = nullptr;

    // step scratch
    int32_t *ids = nullptr, *labels = nullptr;
    float* x_final = nullptr;        // residual after the last layer [T,H]
    mft::bf16* hf = nullptr;         // final-norm output [T,H]
    float *rstd_f = nullptr, *mean_f = nullptr;
    float* dx = nullptr;             // running gradient of the residual stream [T,H] f32
    mft::bf16 *t_h = nullptr, *t_i = nullptr, *t_gu = nullptr, *t_o = nullptr, *t_qk = nullptr, *t_qkv = nullptr, *t_pan = nullptr;
    float *attn_delta = nullptr;
    float* attn_dkv_acc = nullptr;   // f32 [2][T, n_kv, hd]: per-head dK/dV contributions are added here (grouped-query models)
    float* loss_dev = nullptr; int32_t* n_valid_dev = nullptr; float* ce_lse = nullptr; int32_t* status_dev = nullptr;
    void* ce_ws = nullptr; int64_t ce_ws_bytes = 0;
    // Gated MLP: the gating's backward runs in the epilogue of the down-projection dX GEMM, its forward in the epilogue
    // of the gate|up GEMM (three boxes per 64 columns: gate, up, f(gate) * up).  With two epilogue warps per
    // tensor-memory quadrant the fused forward costs 0.54 ms against 0.46 + 0.11 ms for GEMM + activation kernel at
    // Gemma-3-1B widths (with one warp per quadrant it was 0.77 ms).  MFT_FUSE_GLU=0: separate kernels, 1: backward only.
    bool fuse_glu = true, fuse_glu_fwd = true;
    bool fuse_norms = true;          // Gemma: post-norm + residual + pre-norm pairs in one kernel (MFT_FUSE_NORMS=0: separate calls)
    bool ce_onepass = true;          // training steps use mft_lmhead_ce_fused (MFT_CE_ONEPASS=0 selects the two-sweep pair)
    float* stage_f32 = nullptr; int64_t stage_floats = 0;   // upload staging
};
