// Forward / backward / optimizer schedules of the step engine: one stream, a
// fixed sequence of launches per layer, every kernel called through the C ABI
// of mft_cuda.h.  Order of operations follows the reference graphs
// (graph/gemma_model.cpp:358-646, graph/qwen_model.cpp:278-394,
// graph/gpt2_model.cpp:494-764) with the fusions listed next to each call.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "engine.h"

using namespace mft;

namespace {

#define TRY(expr)                         \
    do {                                  \
        int32_t s__ = (expr);             \
        if (s__ != MFT_OK) return s__;    \
    } while (0)

struct Ctx {
    mft_model* m;
    int64_t B, S, T;
    mft_stream_t st;
    float lora_scale;
    mft::DepLaunchScope dep;       // programmatic dependent launch for this call's kernels when the step is small
};

// Columns of the 64-wide LoRA panels that the products read: the rank columns in use, rounded up to the MMA's K step.
// The panel products are asked for just these columns: the tensor map of the 64-row weight panel then ends after them,
// the rest of the tile is filled with zeros by the TMA unit without touching memory, and these HBM-bound launches
// move a third less (x A at rank 16: 16 KB of x and 2 instead of 8 KB of panel per k-block).
inline int64_t panel_cols(const LinearGroup& g) { return (g.k2 + 15) / 16 * 16; }

// y[T, n_total] = x W (+ bias) + scale (x A) B for every linear of the group, one GEMM
// (plus the 64-column x A panel product when the group carries LoRA).
int32_t group_fwd(const Ctx& c, LinearGroup& g, const bf16* x, bf16* xa, bf16* y) {
    if (g.any_lora && !c.m->merged) {
        TRY(mft_gemm_nt(x, g.in, g.a_nk, g.in, c.T, panel_cols(g), g.in, nullptr, 0, nullptr, 0, 0, nullptr, c.lora_scale, xa, 64, MFT_BF16, 0, c.st));
        return mft_gemm_nt(x, g.in, g.w_nk, g.in, c.T, g.n_total, g.in, xa, 64, g.b_nk, 64, g.k2, g.bias, 1.0f, y, g.n_total, MFT_BF16, 0, c.st);
    }
    return mft_gemm_nt(x, g.in, g.w_nk, g.in, c.T, g.n_total, g.in, nullptr, 0, nullptr, 0, 0, g.bias, 1.0f, y, g.n_total, MFT_BF16, 0, c.st);
}

// Gated MLP, forward: gate|up projection with f(gate) * up formed in the GEMM's epilogue; falls back to the GEMM
// followed by the activation kernel when the shape does not qualify.
int32_t glu_fwd(const Ctx& c, LinearGroup& g, int kind, int I, const bf16* x, bf16* xa, bf16* gu, bf16* act) {
    if (c.m->fuse_glu_fwd) {
        const bool lora = g.any_lora && !c.m->merged;
        if (lora) TRY(mft_gemm_nt(x, g.in, g.a_nk, g.in, c.T, panel_cols(g), g.in, nullptr, 0, nullptr, 0, 0, nullptr, c.lora_scale, xa, 64, MFT_BF16, 0, c.st));
        const int32_t s = mft_glu_linear_fwd(kind, x, g.in, g.w_nk, g.in, c.T, I, g.in, lora ? xa : nullptr, 64, lora ? g.b_nk : nullptr, 64, lora ? g.k2 : 0,
                                             g.bias, gu, 2 * I, act, I, c.st);
        if (s != MFT_ERR_UNSUPPORTED) return s;
    }
    TRY(group_fwd(c, g, x, xa, gu));
    return mft_act_fwd(kind, gu, gu + I, 2 * I, act, c.T, I, c.st);
}

// What the backward of a gated MLP hands to group_bwd of the down projection: instead of d(act) the GEMM's epilogue
// writes d_gate|d_up from the saved gate|up.
struct GluBwd {
    int kind, inter;
    const bf16* gu;      // saved gate|up [T, 2*inter]
    bf16* dgu;           // out: d_gate|d_up [T, 2*inter]
    bf16* d_act;         // scratch [T, inter] for the unfused fallback
};

// dx = dy W^T + scale (dy B^T) A^T ; dA-panel += x^T (scale dy B^T) ; dB-panel += (scale x A)^T dy.
int32_t group_bwd(const Ctx& c, LinearGroup& g, const bf16* dy, const bf16* x, const bf16* xa, bf16* dx, bool lora_grads, const GluBwd* glu = nullptr) {
    // dx of a gated MLP's down projection: fused with the gating's backward when possible
    auto dx_gemm = [&](const bf16* gb) -> int32_t {
        if (glu) {
            if (c.m->fuse_glu) {
                const int32_t s = mft_glu_linear_bwd(glu->kind, dy, g.n_total, g.w_kn, g.n_total, c.T, glu->inter, g.n_total, gb, 64, gb ? g.a_kn : nullptr, 64,
                                                     gb ? g.k2 : 0, glu->gu, 2 * glu->inter, glu->dgu, 2 * glu->inter, c.st);
                if (s != MFT_ERR_UNSUPPORTED) return s;
            }
            TRY(mft_gemm_nt(dy, g.n_total, g.w_kn, g.n_total, c.T, g.in, g.n_total, gb, 64, gb ? g.a_kn : nullptr, 64, gb ? g.k2 : 0, nullptr, 1.0f, glu->d_act,
                            g.in, MFT_BF16, 0, c.st));
            return mft_act_bwd(glu->kind, glu->d_act, glu->gu, glu->gu + glu->inter, 2 * glu->inter, glu->dgu, glu->dgu + glu->inter, c.T, glu->inter, c.st);
        }
        return mft_gemm_nt(dy, g.n_total, g.w_kn, g.n_total, c.T, g.in, g.n_total, gb, 64, gb ? g.a_kn : nullptr, 64, gb ? g.k2 : 0, nullptr, 1.0f, dx, g.in,
                           MFT_BF16, 0, c.st);
    };
    if (g.any_lora) {
        bf16* gb = c.m->t_pan;
        TRY(mft_gemm_nt(dy, g.n_total, g.b_kn, g.n_total, c.T, panel_cols(g), g.n_total, nullptr, 0, nullptr, 0, 0, nullptr, c.lora_scale, gb, 64, MFT_BF16, 0, c.st));
        if (dx || glu) TRY(dx_gemm(gb));
        if (lora_grads) {
            // only the rank columns in use (rounded up to 16) of the 64-wide panels take part
            const int rq = (int)panel_cols(g);
            TRY(mft_gemm_tn_acc(x, g.in, gb, 64, c.T, g.in, rq, 1.0f, g.da_pan, 64, c.st));
            TRY(mft_gemm_tn_acc(xa, 64, dy, g.n_total, c.T, rq, g.n_total, 1.0f, g.db_pan, g.n_total, c.st));
        }
        return MFT_OK;
    }
    if (dx || glu) return dx_gemm(nullptr);
    return MFT_OK;
}

mft_strides_t tok_strides(int64_t S, int64_t ld, int64_t hd) {
    mft_strides_t s; s.stride_b = S * ld; s.stride_s = ld; s.stride_h = hd; return s;
}

// Re-packs the bf16 LoRA panels from the f32 masters when an optimizer step or an upload changed them.  Always
// issued on the model's own stream and never inside forward(): forward() may run under stream capture, and a
// pack that depended on this host flag would be frozen into (or left out of) the replayed graph.
int32_t refresh_panels(mft_model* m) {
    if (m->panels_dirty && m->n_pack > 0) {
        TRY(mft_pack_blocks_bf16(m->pack_table, m->n_pack, m->stream));
        m->panels_dirty = false;
    }
    return MFT_OK;
}

int32_t forward(Ctx& c, bool for_training, int64_t n_valid_global = 0) {
    mft_model* m = c.m;
    const mft_model_config_t& cfg = m->cfg;
    const bool gpt2 = cfg.family == MFT_FAMILY_GPT2, gemma = cfg.family == MFT_FAMILY_GEMMA;
    const int H = cfg.hidden, I = cfg.inter, nh = cfg.n_heads, nkv = cfg.n_kv_heads, hd = cfg.head_dim, L = cfg.layers;
    const int QD = nh * hd, KD = nkv * hd, QKV = QD + 2 * KD;
    const int64_t T = c.T, S = c.S;
    (void)for_training;
    const bool fuse = gemma && m->fuse_norms && H <= 2048;      // Gemma's post-norm + residual + pre-norm pairs in one kernel
    TRY(mft_memset(m->status_dev, 0, 4, c.st));
    const float emb_scale = gemma ? std::sqrt((float)H) : 1.0f;
    TRY(mft_embedding_gather(m->ids, m->embed, gpt2 ? m->pos_embed : nullptr, m->bufs[0].x, T, S, H, cfg.vocab, emb_scale, m->status_dev, c.st));

    for (int l = 0; l < L; ++l) {
        LayerWeights& w = m->layers[l];
        LayerBuffers& b = m->bufs[l];
        float* x_next = (l + 1 < L) ? m->bufs[l + 1].x : m->x_final;
        // ---- attention block
        if (gpt2) TRY(mft_layernorm_fwd(b.x, MFT_F32, w.ln1_w, w.ln1_b, 1e-5f, b.h1, MFT_BF16, b.mean1, b.rstd1, T, H, c.st));
        else if (!(fuse && l > 0))     // with fused norms the previous layer's last kernel already produced h1 / rstd1
            TRY(mft_rmsnorm_fwd(b.x, MFT_F32, w.ln1_w, cfg.norm_eps, gemma ? 1 : 0, b.h1, MFT_BF16, b.rstd1, nullptr, nullptr, T, H, c.st));
        TRY(group_fwd(c, w.qkv, b.h1, b.xa_qkv, b.qkv));
        const bf16 *q, *k, *v = b.qkv + QD + KD;
        int64_t ldqk;
        if (gpt2) { q = b.qkv; k = b.qkv + QD; ldqk = QKV; }
        else {
            const float* cs = (gemma && w.sliding) ? m->cos_l : m->cos_g;
            const float* sn = (gemma && w.sliding) ? m->sin_l : m->sin_g;
            // per-head RMSNorm (Gemma) fused with the rotary embedding and the head split
            TRY(mft_headnorm_rope_fwd(b.qkv, QKV, gemma ? w.q_norm_w : nullptr, cfg.norm_eps, cs, sn, b.qk_r, QD + KD, b.rstd_q, T, S, nh, hd, c.st));
            TRY(mft_headnorm_rope_fwd(b.qkv + QD, QKV, gemma ? w.k_norm_w : nullptr, cfg.norm_eps, cs, sn, b.qk_r + QD, QD + KD, b.rstd_k, T, S, nkv, hd, c.st));
            q = b.qk_r; k = b.qk_r + QD; ldqk = QD + KD;
        }
        const int64_t window = (gemma && w.sliding) ? cfg.sliding_window : 0;
        TRY(mft_attn_fwd(q, tok_strides(S, ldqk, hd), k, tok_strides(S, ldqk, hd), v, tok_strides(S, QKV, hd), b.o, tok_strides(S, QD, hd),
                         b.lse, c.B, S, nh, nkv, hd, cfg.attn_scale, window, c.st));
        TRY(group_fwd(c, w.o, b.o, b.xa_o, b.attn_out));
        if (fuse) {
            // x_mid = x + rms_norm(attn_out) and the pre-feedforward norm of x_mid, one pass per row
            TRY(mft_rmsnorm_add_norm_fwd(b.attn_out, w.post_attn_w, 1, b.x, w.ln2_w, 1, cfg.norm_eps, b.x_mid, b.rstd2, b.h2, b.rstd3, T, H, c.st));
        } else if (gemma) {
            // x_mid = x + rms_norm(attn_out) in one pass, then the pre-feedforward norm
            TRY(mft_rmsnorm_fwd(b.attn_out, MFT_BF16, w.post_attn_w, cfg.norm_eps, 1, nullptr, MFT_BF16, b.rstd2, b.x, b.x_mid, T, H, c.st));
            TRY(mft_rmsnorm_fwd(b.x_mid, MFT_F32, w.ln2_w, cfg.norm_eps, 1, b.h2, MFT_BF16, b.rstd3, nullptr, nullptr, T, H, c.st));
        } else {
            TRY(mft_add_f32_bf16(b.x, b.attn_out, b.x_mid, T * H, c.st));
            if (gpt2) TRY(mft_layernorm_fwd(b.x_mid, MFT_F32, w.ln2_w, w.ln2_b, 1e-5f, b.h2, MFT_BF16, b.mean3, b.rstd3, T, H, c.st));
            else TRY(mft_rmsnorm_fwd(b.x_mid, MFT_F32, w.ln2_w, cfg.norm_eps, 0, b.h2, MFT_BF16, b.rstd3, nullptr, nullptr, T, H, c.st));
        }
        // ---- MLP block
        if (gpt2) {
            TRY(group_fwd(c, w.gu, b.h2, b.xa_gu, b.gu));
            TRY(mft_act_fwd(MFT_ACT_GELU, b.gu, nullptr, I, b.act, T, I, c.st));
        } else {
            TRY(glu_fwd(c, w.gu, gemma ? MFT_ACT_GEGLU : MFT_ACT_SWIGLU, I, b.h2, b.xa_gu, b.gu, b.act));
        }
        TRY(group_fwd(c, w.down, b.act, b.xa_d, b.mlp_out));
        if (fuse) {
            // x_next = x_mid + rms_norm(mlp_out) and the norm that reads x_next: the next layer's input norm, or the final norm
            const bool last = l + 1 == L;
            TRY(mft_rmsnorm_add_norm_fwd(b.mlp_out, w.post_ffn_w, 1, b.x_mid, last ? m->final_w : m->layers[l + 1].ln1_w, 1, cfg.norm_eps, x_next,
                                         b.rstd4, last ? m->hf : m->bufs[l + 1].h1, last ? m->rstd_f : m->bufs[l + 1].rstd1, T, H, c.st));
        } else if (gemma) TRY(mft_rmsnorm_fwd(b.mlp_out, MFT_BF16, w.post_ffn_w, cfg.norm_eps, 1, nullptr, MFT_BF16, b.rstd4, b.x_mid, x_next, T, H, c.st));
        else TRY(mft_add_f32_bf16(b.x_mid, b.mlp_out, x_next, T * H, c.st));
    }
    if (gpt2) TRY(mft_layernorm_fwd(m->x_final, MFT_F32, m->final_w, m->final_b, 1e-5f, m->hf, MFT_BF16, m->mean_f, m->rstd_f, T, H, c.st));
    else if (!fuse) TRY(mft_rmsnorm_fwd(m->x_final, MFT_F32, m->final_w, cfg.norm_eps, gemma ? 1 : 0, m->hf, MFT_BF16, m->rstd_f, nullptr, nullptr, T, H, c.st));
    // lm head + shifted cross entropy; the [T,V] logits are never written.  A training step gets the loss and
    // d(loss)/d(final hidden) (into t_h) from one sweep over the vocabulary.
    if (for_training && m->ce_onepass)
        return mft_lmhead_ce_fused(m->hf, m->embed, m->embed_t, m->ld_t, m->labels, c.B, S, H, cfg.vocab, -100, n_valid_global, m->loss_scale,
                                   m->loss_dev, m->n_valid_dev, m->ce_lse, m->t_h, m->status_dev, m->ce_ws, m->ce_ws_bytes, c.st);
    return mft_lmhead_ce_fwd(m->hf, m->embed, m->labels, c.B, S, H, cfg.vocab, -100, m->loss_dev, m->n_valid_dev, m->ce_lse, m->status_dev,
                             m->ce_ws, m->ce_ws_bytes, c.st);
}

int32_t backward(Ctx& c, int64_t n_valid_global) {
    mft_model* m = c.m;
    const mft_model_config_t& cfg = m->cfg;
    const bool gpt2 = cfg.family == MFT_FAMILY_GPT2, gemma = cfg.family == MFT_FAMILY_GEMMA;
    const bool detach = gpt2 && cfg.gpt2_detach_attn != 0;
    const int H = cfg.hidden, I = cfg.inter, nh = cfg.n_heads, nkv = cfg.n_kv_heads, hd = cfg.head_dim, L = cfg.layers;
    const int QD = nh * hd, KD = nkv * hd, QKV = QD + 2 * KD;
    const int64_t T = c.T, S = c.S;
    if (m->grad_pan_floats > 0) TRY(mft_memset(m->grad_pan_base, 0, (size_t)m->grad_pan_floats * 4, c.st));
    // d(loss)/d(final hidden), then through the final norm into the residual gradient dx (f32)
    if (!m->ce_onepass)
        TRY(mft_lmhead_ce_bwd(m->hf, m->embed, m->embed_t, m->ld_t, m->labels, c.B, S, H, cfg.vocab, -100, m->ce_lse, m->n_valid_dev,
                              n_valid_global, m->loss_scale, m->t_h, m->ce_ws, m->ce_ws_bytes, c.st));
    if (gpt2) TRY(mft_layernorm_bwd(m->t_h, MFT_BF16, m->x_final, MFT_F32, m->final_w, m->mean_f, m->rstd_f, m->dx, MFT_F32, 0, nullptr, nullptr, T, H, c.st));
    else TRY(mft_rmsnorm_bwd(m->t_h, MFT_BF16, m->x_final, MFT_F32, m->final_w, m->rstd_f, cfg.norm_eps, gemma ? 1 : 0, m->dx, MFT_F32, 0, nullptr, T, H, c.st));

    const bool fuse = gemma && m->fuse_norms && H <= 2048;
    bool have_d_mlp_out = false;
    for (int l = L - 1; l >= 0; --l) {
        LayerWeights& w = m->layers[l];
        LayerBuffers& b = m->bufs[l];
        // ---- MLP block: dx is d(loss)/d(x_next) on entry
        const bf16* d_mlp_out;
        if (gemma) {
            // (with fused norms the layer above already pushed dx through this layer's post-feedforward norm into t_h)
            if (!have_d_mlp_out)
                TRY(mft_rmsnorm_bwd(m->dx, MFT_F32, b.mlp_out, MFT_BF16, w.post_ffn_w, b.rstd4, cfg.norm_eps, 1, m->t_h, MFT_BF16, 0, nullptr, T, H, c.st));
            have_d_mlp_out = false;
        } else {
            TRY(mft_cast_f32_to_bf16(m->dx, m->t_h, T * H, c.st));
        }
        d_mlp_out = m->t_h;
        if (gpt2) {
            TRY(group_bwd(c, w.down, d_mlp_out, b.act, b.xa_d, m->t_i, true));
            TRY(mft_act_bwd(MFT_ACT_GELU, m->t_i, b.gu, nullptr, I, m->t_gu, nullptr, T, I, c.st));
        } else {
            const GluBwd glu{gemma ? MFT_ACT_GEGLU : MFT_ACT_SWIGLU, I, b.gu, m->t_gu, m->t_i};
            TRY(group_bwd(c, w.down, d_mlp_out, b.act, b.xa_d, nullptr, true, &glu));
        }
        TRY(group_bwd(c, w.gu, m->t_gu, b.h2, b.xa_gu, m->t_h, true));
        // through the pre-MLP norm, accumulated onto the residual gradient: dx = d(loss)/d(x_mid)
        if (gpt2) TRY(mft_layernorm_bwd(m->t_h, MFT_BF16, b.x_mid, MFT_F32, w.ln2_w, b.mean3, b.rstd3, m->dx, MFT_F32, 1, nullptr, nullptr, T, H, c.st));
        else if (fuse)   // pre-feedforward norm (adds into dx) and post-attention norm (dx -> t_h) in one pass per row
            TRY(mft_rmsnorm_pair_bwd(m->t_h, b.x_mid, w.ln2_w, 1, b.rstd3, m->dx, b.attn_out, w.post_attn_w, 1, b.rstd2, m->t_h, T, H, c.st));
        else TRY(mft_rmsnorm_bwd(m->t_h, MFT_BF16, b.x_mid, MFT_F32, w.ln2_w, b.rstd3, cfg.norm_eps, gemma ? 1 : 0, m->dx, MFT_F32, 1, nullptr, T, H, c.st));
        // ---- attention block
        if (fuse) {}
        else if (gemma) TRY(mft_rmsnorm_bwd(m->dx, MFT_F32, b.attn_out, MFT_BF16, w.post_attn_w, b.rstd2, cfg.norm_eps, 1, m->t_h, MFT_BF16, 0, nullptr, T, H, c.st));
        else TRY(mft_cast_f32_to_bf16(m->dx, m->t_h, T * H, c.st));
        if (detach) {
            // Reference-parity GPT-2: the QKV split severs autograd, so c_proj gets its LoRA gradients
            // (its input is a constant) and nothing flows back through attention, c_attn or ln_1.
            TRY(group_bwd(c, w.o, m->t_h, b.o, b.xa_o, nullptr, true));
            continue;
        }
        TRY(group_bwd(c, w.o, m->t_h, b.o, b.xa_o, m->t_o, true));
        const bf16 *q, *k, *v = b.qkv + QD + KD;
        int64_t ldqk;
        bf16 *dq, *dk, *dv = m->t_qkv + QD + KD;
        if (gpt2) { q = b.qkv; k = b.qkv + QD; ldqk = QKV; dq = m->t_qkv; dk = m->t_qkv + QD; }
        else { q = b.qk_r; k = b.qk_r + QD; ldqk = QD + KD; dq = m->t_qk; dk = m->t_qk + QD; }
        const int64_t window = (gemma && w.sliding) ? cfg.sliding_window : 0;
        TRY(mft_attn_bwd(q, tok_strides(S, ldqk, hd), k, tok_strides(S, ldqk, hd), v, tok_strides(S, QKV, hd), b.o, tok_strides(S, QD, hd),
                         m->t_o, tok_strides(S, QD, hd), b.lse, dq, dk, dv, m->attn_delta, m->attn_dkv_acc, c.B, S, nh, nkv, hd, cfg.attn_scale, window, c.st));
        if (!gpt2) {
            const float* cs = (gemma && w.sliding) ? m->cos_l : m->cos_g;
            const float* sn = (gemma && w.sliding) ? m->sin_l : m->sin_g;
            TRY(mft_headnorm_rope_bwd(m->t_qk, QD + KD, b.qkv, QKV, gemma ? w.q_norm_w : nullptr, b.rstd_q, cs, sn, m->t_qkv, QKV, T, S, nh, hd, c.st));
            TRY(mft_headnorm_rope_bwd(m->t_qk + QD, QD + KD, b.qkv + QD, QKV, gemma ? w.k_norm_w : nullptr, b.rstd_k, cs, sn, m->t_qkv + QD, QKV, T, S, nkv, hd, c.st));
        }
        const bool need_dx = l > 0;   // the embedding table is frozen: layer 0 needs no input gradient
        TRY(group_bwd(c, w.qkv, m->t_qkv, b.h1, b.xa_qkv, need_dx ? m->t_h : nullptr, true));
        if (need_dx) {
            if (gpt2) TRY(mft_layernorm_bwd(m->t_h, MFT_BF16, b.x, MFT_F32, w.ln1_w, b.mean1, b.rstd1, m->dx, MFT_F32, 1, nullptr, nullptr, T, H, c.st));
            else if (fuse) {
                // this layer's input norm (adds into dx) and the post-feedforward norm of the layer below (dx -> t_h)
                TRY(mft_rmsnorm_pair_bwd(m->t_h, b.x, w.ln1_w, 1, b.rstd1, m->dx, m->bufs[l - 1].mlp_out, m->layers[l - 1].post_ffn_w, 1,
                                         m->bufs[l - 1].rstd4, m->t_h, T, H, c.st));
                have_d_mlp_out = true;
            } else TRY(mft_rmsnorm_bwd(m->t_h, MFT_BF16, b.x, MFT_F32, w.ln1_w, b.rstd1, cfg.norm_eps, gemma ? 1 : 0, m->dx, MFT_F32, 1, nullptr, T, H, c.st));
        }
    }
    if (m->n_unpack > 0) TRY(mft_accumulate_blocks_f32(m->unpack_table, m->n_unpack, c.st));
    return MFT_OK;
}

int32_t make_ctx(mft_model* m, int32_t batch, int32_t seq, Ctx* c) {
    MFT_CHECK_ARG(m && batch > 0 && seq > 1, "step: bad batch/seq");
    MFT_CHECK_ARG((int64_t)batch * seq <= m->max_tokens && seq <= m->cfg.max_seq, "step: batch*seq exceeds the model's capacity");
    c->m = m; c->B = batch; c->S = seq; c->T = (int64_t)batch * seq; c->st = m->stream;
    c->lora_scale = m->cfg.lora_rank > 0 ? m->cfg.lora_alpha / (float)m->cfg.lora_rank : 0.f;
    c->dep.set(c->T <= 8192);
    return MFT_OK;
}

int32_t check_status(mft_model* m) {
    int32_t st = 0;
    TRY(mft_memcpy_d2h(&st, m->status_dev, 4, m->stream));
    if (st == MFT_ERR_BOUNDS) return fail(MFT_ERR_BOUNDS, "token id or label out of range");
    int32_t dev = 0;
    TRY(mft_device_status(m->stream, &dev));
    if (dev != 0) return fail(dev, "a kernel wait ran out (device status word set)");
    return MFT_OK;
}

// Forward + backward of a training step.  The second call with the same (batch, seq, n_valid_global) captures the
// launches into a CUDA graph on the model's private stream; later calls replay it.  Anything that prevents a
// capture (a profiling hook, a failing call) falls back to issuing the launches directly.
int32_t forward_backward(Ctx& c, int64_t n_valid_global) {
    mft_model* m = c.m;
    if (m->merged) return fail(MFT_ERR_INVALID_ARG, "the adapters are merged into the base weights: call mft_model_unmerge_lora before training");
    TRY(refresh_panels(m));
    auto eager = [&]() -> int32_t {
        TRY(forward(c, true, n_valid_global));
        return backward(c, n_valid_global);
    };
    if (!m->use_graph || gemm_profiling_enabled()) return eager();
    StepGraph* g = nullptr;
    for (auto& e : m->graphs)
        if (e.batch == c.B && e.seq == c.S && e.n_valid_global == n_valid_global && e.loss_scale == m->loss_scale) { g = &e; break; }
    if (!g) {
        if (m->graphs.size() >= 8) return eager();         // the key keeps changing (e.g. varying global counts): do not hoard graphs
        m->graphs.push_back(StepGraph{c.B, c.S, n_valid_global, m->loss_scale, 0, 0, nullptr});
        g = &m->graphs.back();
    }
    if (!g->exec) {
        if (g->calls++ == 0) return eager();                // first run: one-time attribute set-up happens outside any capture
        if (!m->graph_stream) {
            if (cudaStreamCreateWithFlags(&m->graph_stream, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&m->graph_in, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&m->graph_out, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                m->use_graph = false;
                return eager();
            }
        }
        Ctx cc;                                 // the same call on the capture stream (the launch hint stays c's)
        cc.m = c.m; cc.B = c.B; cc.S = c.S; cc.T = c.T; cc.lora_scale = c.lora_scale;
        cc.st = m->graph_stream;
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(m->graph_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            m->use_graph = false;
            return eager();
        }
        const int64_t launches_before = mft_launch_count();
        int32_t s = forward(cc, true, n_valid_global);
        if (s == MFT_OK) s = backward(cc, n_valid_global);
        g->kernels = mft_launch_count() - launches_before;
        count_launch(-(int)g->kernels);                      // captured, not run: counted at every replay instead
        const cudaError_t ce = cudaStreamEndCapture(m->graph_stream, &graph);
        if (s != MFT_OK || ce != cudaSuccess || !graph || cudaGraphInstantiate(&g->exec, graph, 0) != cudaSuccess) {
            cudaGetLastError();
            if (graph) cudaGraphDestroy(graph);
            g->exec = nullptr;
            m->use_graph = false;
            return eager();
        }
        cudaGraphDestroy(graph);
    }
    // order the replay after what the caller queued on its stream, and the caller's stream after the replay
    if (int32_t s = check_cuda(cudaEventRecord(m->graph_in, m->stream), "step graph event")) return s;
    if (int32_t s = check_cuda(cudaStreamWaitEvent(m->graph_stream, m->graph_in, 0), "step graph wait")) return s;
    if (int32_t s = check_cuda(cudaGraphLaunch(g->exec, m->graph_stream), "step graph launch")) return s;
    count_launch((int)g->kernels);
    if (int32_t s = check_cuda(cudaEventRecord(m->graph_out, m->graph_stream), "step graph event")) return s;
    return check_cuda(cudaStreamWaitEvent(m->stream, m->graph_out, 0), "step graph wait");
}

}  // namespace

extern "C" int32_t mft_model_forward_backward_dev(mft_model_t* m, const int32_t* ids_dev, const int32_t* labels_dev, int32_t batch,
                                                  int32_t seq, int64_t n_valid_global, float** loss_dev, int32_t** n_valid_dev) {
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    MFT_CHECK_ARG(ids_dev && labels_dev, "mft_model_forward_backward_dev: null input");
    if (ids_dev != m->ids) TRY(mft_memcpy_d2d(m->ids, ids_dev, (size_t)c.T * 4, c.st));
    if (labels_dev != m->labels) TRY(mft_memcpy_d2d(m->labels, labels_dev, (size_t)c.T * 4, c.st));
    TRY(forward_backward(c, n_valid_global));
    if (loss_dev) *loss_dev = m->loss_dev;
    if (n_valid_dev) *n_valid_dev = m->n_valid_dev;
    return MFT_OK;
}

extern "C" int32_t mft_model_forward_backward(mft_model_t* m, const int32_t* ids_host, const int32_t* labels_host, int32_t batch,
                                              int32_t seq, int64_t n_valid_global, float* loss_host, int32_t* n_valid_host) {
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    MFT_CHECK_ARG(ids_host && labels_host, "mft_model_forward_backward: null input");
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, labels_host, (size_t)c.T * 4, c.st));
    TRY(forward_backward(c, n_valid_global));
    if (loss_host) TRY(mft_memcpy_d2h(loss_host, m->loss_dev, 4, c.st));
    if (n_valid_host) TRY(mft_memcpy_d2h(n_valid_host, m->n_valid_dev, 4, c.st));
    return check_status(m);
}

extern "C" int32_t mft_model_forward_loss(mft_model_t* m, const int32_t* ids_host, const int32_t* labels_host, int32_t batch,
                                          int32_t seq, float* loss_host) {
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    MFT_CHECK_ARG(ids_host && labels_host && loss_host, "mft_model_forward_loss: null argument");
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, labels_host, (size_t)c.T * 4, c.st));
    TRY(refresh_panels(m));
    TRY(forward(c, false));
    TRY(mft_memcpy_d2h(loss_host, m->loss_dev, 4, c.st));
    return check_status(m);
}

// Dense logits of the positions computed by the last forward pass: out[t, v] = hidden_final[t, :] . table[v, :]
// (f32 [batch*seq, vocab]).  Only for callers that insist on the materialised [B,S,V] tensor; training and
// evaluation never form it.
extern "C" int32_t mft_model_forward_logits(mft_model_t* m, const int32_t* ids_host, int32_t batch, int32_t seq, float* logits_dev) {
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    MFT_CHECK_ARG(ids_host && logits_dev, "mft_model_forward_logits: null argument");
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, ids_host, (size_t)c.T * 4, c.st));      // any valid labels: the loss is not used
    TRY(refresh_panels(m));
    TRY(forward(c, false));
    TRY(mft_gemm_nt(m->hf, m->cfg.hidden, m->embed, m->cfg.hidden, c.T, m->cfg.vocab, m->cfg.hidden, nullptr, 0, nullptr, 0, 0, nullptr, 1.0f,
                    logits_dev, m->cfg.vocab, MFT_F32, 0, c.st));
    return check_status(m);
}

// The final-norm output of a forward pass as f32 [batch*seq, hidden] on the device (QwenModel::forward_hidden).
extern "C" int32_t mft_model_forward_hidden(mft_model_t* m, const int32_t* ids_host, int32_t batch, int32_t seq, float* hidden_dev) {
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    MFT_CHECK_ARG(ids_host && hidden_dev, "mft_model_forward_hidden: null argument");
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, ids_host, (size_t)c.T * 4, c.st));
    TRY(refresh_panels(m));
    TRY(forward(c, false));
    TRY(mft_cast_bf16_to_f32(m->hf, hidden_dev, c.T * m->cfg.hidden, c.st));
    return check_status(m);
}

// ---------------------------------------------------------------- double-buffered input
static int32_t ensure_slots(mft_model* m) {
    if (m->copy_stream) return MFT_OK;
    if (int32_t s = check_cuda(cudaStreamCreateWithFlags(&m->copy_stream, cudaStreamNonBlocking), "copy stream")) return s;
    for (int i = 0; i < 2; ++i) {
        void* p = nullptr;
        TRY(mft_malloc((size_t)m->max_tokens * 4, m->stream, &p)); m->slot_ids[i] = static_cast<int32_t*>(p); m->allocations.push_back(p);
        TRY(mft_malloc((size_t)m->max_tokens * 4, m->stream, &p)); m->slot_labels[i] = static_cast<int32_t*>(p); m->allocations.push_back(p);
        if (int32_t s = check_cuda(cudaEventCreateWithFlags(&m->slot_ready[i], cudaEventDisableTiming), "slot event")) return s;
        if (int32_t s = check_cuda(cudaEventCreateWithFlags(&m->slot_free[i], cudaEventDisableTiming), "slot event")) return s;
    }
    return MFT_OK;
}

extern "C" int32_t mft_model_stage_batch(mft_model_t* m, int32_t slot, const int32_t* ids_pinned, const int32_t* labels_pinned,
                                         int32_t batch, int32_t seq) {
    MFT_CHECK_ARG(m && (slot == 0 || slot == 1) && ids_pinned && labels_pinned, "mft_model_stage_batch: bad argument");
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    TRY(ensure_slots(m));
    // the step that last consumed this slot must have copied it out before it is overwritten
    if (int32_t s = check_cuda(cudaStreamWaitEvent(m->copy_stream, m->slot_free[slot], 0), "slot wait")) return s;
    TRY(mft_memcpy_h2d(m->slot_ids[slot], ids_pinned, (size_t)c.T * 4, m->copy_stream));
    TRY(mft_memcpy_h2d(m->slot_labels[slot], labels_pinned, (size_t)c.T * 4, m->copy_stream));
    return check_cuda(cudaEventRecord(m->slot_ready[slot], m->copy_stream), "slot event");
}

extern "C" int32_t mft_model_stage_wait(mft_model_t* m, int32_t slot) {
    MFT_CHECK_ARG(m && (slot == 0 || slot == 1) && m->copy_stream, "mft_model_stage_wait: nothing was staged");
    return check_cuda(cudaEventSynchronize(m->slot_ready[slot]), "slot wait");
}

extern "C" int32_t mft_model_step_staged(mft_model_t* m, int32_t slot, int32_t batch, int32_t seq, int64_t n_valid_global,
                                         float* loss_pinned, int32_t* n_valid_pinned) {
    MFT_CHECK_ARG(m && (slot == 0 || slot == 1) && m->copy_stream, "mft_model_step_staged: nothing was staged");
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    if (int32_t s = check_cuda(cudaStreamWaitEvent(m->stream, m->slot_ready[slot], 0), "slot wait")) return s;
    TRY(mft_memcpy_d2d(m->ids, m->slot_ids[slot], (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_d2d(m->labels, m->slot_labels[slot], (size_t)c.T * 4, c.st));
    if (int32_t s = check_cuda(cudaEventRecord(m->slot_free[slot], m->stream), "slot event")) return s;
    TRY(forward_backward(c, n_valid_global));
    if (loss_pinned)
        if (int32_t s = check_cuda(cudaMemcpyAsync(loss_pinned, m->loss_dev, 4, cudaMemcpyDeviceToHost, m->stream), "loss copy")) return s;
    if (n_valid_pinned)
        if (int32_t s = check_cuda(cudaMemcpyAsync(n_valid_pinned, m->n_valid_dev, 4, cudaMemcpyDeviceToHost, m->stream), "count copy")) return s;
    return MFT_OK;
}

extern "C" int32_t mft_model_sync(mft_model_t* m) {
    MFT_CHECK_ARG(m, "mft_model_sync: null model");
    if (int32_t s = check_cuda(cudaStreamSynchronize(m->stream), "model sync")) return s;
    return check_status(m);
}

extern "C" int32_t mft_model_eval_ppl_batch(mft_model_t* m, mft_ppl_accum_t* acc, const int32_t* ids_host, const int32_t* labels_host,
                                            int32_t batch, int32_t seq) {
    MFT_CHECK_ARG(m && acc && ids_host && labels_host, "mft_model_eval_ppl_batch: null argument");
    float loss_val = 0.f;
    TRY(mft_model_forward_loss(m, ids_host, labels_host, batch, seq, &loss_val));
    int64_t valid = 0;
    for (int64_t i = 0; i < (int64_t)batch * seq; ++i)
        if (labels_host[i] != -100) valid++;
    acc->sum_loss += loss_val * valid;      // float * int64 -> float, then widened: the reference's expression
    acc->sum_tokens += valid;
    acc->n_batches += 1;
    return MFT_OK;
}

extern "C" int32_t mft_ppl_result(const mft_ppl_accum_t* acc, float* mean_nll, float* ppl) {
    MFT_CHECK_ARG(acc && mean_nll && ppl, "mft_ppl_result: null argument");
    *mean_nll = acc->sum_tokens > 0 ? (float)(acc->sum_loss / (double)acc->sum_tokens) : 0.0f;
    *ppl = std::exp(*mean_nll);
    return MFT_OK;
}

extern "C" int32_t mft_model_score_tokens(mft_model_t* m, const int32_t* ids_host, int32_t seq, const int32_t* cand_host,
                                          int32_t n_cand, float* logprob_host) {
    MFT_CHECK_ARG(m && ids_host && cand_host && logprob_host && n_cand > 0 && n_cand <= 64, "mft_model_score_tokens: bad argument");
    Ctx c;
    TRY(make_ctx(m, 1, seq, &c));
    const int64_t H = m->cfg.hidden, V = m->cfg.vocab;
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)seq * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, ids_host, (size_t)seq * 4, c.st));      // any valid labels: the loss is not used
    TRY(refresh_panels(m));
    TRY(forward(c, false));
    // scratch inside the staging buffer: candidate rows (f32, then bf16), the last hidden row twice, logits, ids
    MFT_CHECK_ARG((64 + 2) * H * 2 + 1024 <= m->stage_floats - 64, "mft_model_score_tokens: staging buffer too small");
    float* rows_f32 = m->stage_f32;
    bf16* rows_bf16 = reinterpret_cast<bf16*>(rows_f32 + 64 * H);
    bf16* pair = rows_bf16 + 64 * H;
    float* logits = reinterpret_cast<float*>(pair + 2 * H + 64);
    float* lse = logits + 64;
    float* loss_tmp = lse + 8;
    int32_t* ints = reinterpret_cast<int32_t*>(loss_tmp + 8);                 // cand[64], labels2[2], n_valid[1]
    int32_t cand_clean[64], labels2[2] = {0, 0};
    for (int i = 0; i < n_cand; ++i) cand_clean[i] = (cand_host[i] >= 0 && cand_host[i] < V) ? cand_host[i] : 0;
    TRY(mft_memcpy_h2d(ints, cand_clean, (size_t)n_cand * 4, c.st));
    TRY(mft_memcpy_h2d(ints + 64, labels2, 8, c.st));
    TRY(mft_embedding_gather(ints, m->embed, nullptr, rows_f32, n_cand, 1, H, V, 1.0f, m->status_dev, c.st));
    TRY(mft_cast_f32_to_bf16(rows_f32, rows_bf16, (int64_t)n_cand * H, c.st));
    const bf16* h_last = m->hf + (int64_t)(seq - 1) * H;
    TRY(mft_memcpy_d2d(pair, h_last, (size_t)H * 2, c.st));
    TRY(mft_memcpy_d2d(pair + H, h_last, (size_t)H * 2, c.st));
    TRY(mft_gemm_nt(h_last, H, rows_bf16, H, 1, n_cand, H, nullptr, 0, nullptr, 0, 0, nullptr, 1.0f, logits, 64, MFT_F32, 0, c.st));
    // log-sum-exp of the last position over the whole vocabulary: row 0 of a 1 x 2 "batch" made of that row twice
    TRY(mft_lmhead_ce_fwd(pair, m->embed, ints + 64, 1, 2, H, V, -100, loss_tmp, ints + 66, lse, m->status_dev, m->ce_ws, m->ce_ws_bytes, c.st));
    float logits_host[64], lse_host = 0.f;
    TRY(mft_memcpy_d2h(logits_host, logits, (size_t)n_cand * 4, c.st));
    TRY(mft_memcpy_d2h(&lse_host, lse, 4, c.st));
    TRY(check_status(m));
    for (int i = 0; i < n_cand; ++i)
        logprob_host[i] = (cand_host[i] >= 0 && cand_host[i] < V) ? logits_host[i] - lse_host : -1e30f;
    return MFT_OK;
}

extern "C" int32_t mft_model_optimizer_step(mft_model_t* m, float lr, float beta1, float beta2, float eps, float weight_decay,
                                            float max_norm, float clip_eps) {
    MFT_CHECK_ARG(m, "mft_model_optimizer_step: null model");
    MFT_CHECK_ARG(!m->merged, "mft_model_optimizer_step: the adapters are merged into the base weights");
    if (m->bucket_n == 0) return MFT_OK;
    m->adam_step += 1;
    const float* sq = nullptr;
    if (max_norm > 0.f) {
        TRY(mft_grad_sqnorm(m->g_bucket, m->bucket_n, m->sqnorm, m->stream));
        sq = m->sqnorm;
    }
    // Tensors the reference never gives a gradient (GPT-2 c_attn) keep a zero gradient and zero Adam
    // moments, so the update leaves them untouched, as Adam::step skips them.
    TRY(mft_adam_step(m->p_bucket, m->g_bucket, m->m_bucket, m->v_bucket, m->bucket_n, m->adam_step, lr, beta1, beta2, eps,
                      weight_decay, sq, max_norm, clip_eps, 1, m->stream));
    m->panels_dirty = true;
    return MFT_OK;
}

extern "C" int32_t mft_model_set_loss_scale(mft_model_t* m, float scale) {
    MFT_CHECK_ARG(m && std::isfinite(scale) && scale != 0.f, "mft_model_set_loss_scale: bad argument");
    m->loss_scale = scale;
    return MFT_OK;
}

// ---------------------------------------------------------------- step driver
struct mft_trainer {
    mft_model* model;
    mft_trainer_config_t cfg;
    int64_t global_step = 0;
    int accum_counter = 0;
    float* loss_acc = nullptr;        // device: sum of the window's micro-batch losses
};

extern "C" float mft_trainer_lr(const mft_trainer_config_t* cfg, int64_t step) {
    if (!cfg) return 0.f;
    // same integer / float arithmetic as get_lr of the trainers
    const int64_t total = std::max<int64_t>(1, cfg->total_updates);
    const int warmup_steps = static_cast<int>(total * cfg->warmup_ratio);
    if (warmup_steps > 0 && step <= warmup_steps) return cfg->learning_rate * (static_cast<float>(step) / warmup_steps);
    float progress = static_cast<float>(step - warmup_steps) / std::max<int64_t>(1, total - warmup_steps);
    progress = std::min(std::max(progress, 0.0f), 1.0f);
    if (cfg->lr_scheduler == MFT_LR_COSINE) return cfg->learning_rate * 0.5f * (1.0f + std::cos(3.14159265f * progress));
    if (cfg->lr_scheduler == MFT_LR_LINEAR) return cfg->learning_rate * (1.0f - progress);
    return cfg->learning_rate;
}

extern "C" int32_t mft_trainer_create(mft_model_t* model, const mft_trainer_config_t* cfg, mft_trainer_t** out) {
    MFT_CHECK_ARG(model && cfg && out, "mft_trainer_create: null argument");
    MFT_CHECK_ARG(cfg->grad_accum_steps >= 1 && cfg->lr_scheduler >= MFT_LR_LINEAR && cfg->lr_scheduler <= MFT_LR_CONSTANT,
                  "mft_trainer_create: bad configuration");
    auto* t = new mft_trainer();
    t->model = model;
    t->cfg = *cfg;
    void* p = nullptr;
    if (int32_t s = mft_malloc(4, model->stream, &p)) { delete t; return s; }
    t->loss_acc = static_cast<float*>(p);
    if (int32_t s = mft_memset(t->loss_acc, 0, 4, model->stream)) { mft_free(p, model->stream); delete t; return s; }
    *out = t;
    return MFT_OK;
}

extern "C" int32_t mft_trainer_destroy(mft_trainer_t* t) {
    if (!t) return MFT_OK;
    cudaStreamSynchronize(t->model->stream);
    mft_free(t->loss_acc, t->model->stream);
    delete t;
    return MFT_OK;
}

extern "C" int64_t mft_trainer_global_step(const mft_trainer_t* t) { return t ? t->global_step : 0; }

extern "C" int32_t mft_trainer_train_step(mft_trainer_t* t, const int32_t* ids_host, const int32_t* labels_host, int32_t batch,
                                          int32_t seq, int64_t n_valid_global, int32_t* stepped, float* avg_loss, float* lr_used) {
    MFT_CHECK_ARG(t && ids_host && labels_host && stepped, "mft_trainer_train_step: null argument");
    mft_model* m = t->model;
    Ctx c;
    TRY(make_ctx(m, batch, seq, &c));
    const float saved_scale = m->loss_scale;
    m->loss_scale = 1.0f / static_cast<float>(t->cfg.grad_accum_steps);
    TRY(mft_memcpy_h2d(m->ids, ids_host, (size_t)c.T * 4, c.st));
    TRY(mft_memcpy_h2d(m->labels, labels_host, (size_t)c.T * 4, c.st));
    const int32_t s = forward_backward(c, n_valid_global);
    m->loss_scale = saved_scale;
    if (s != MFT_OK) return s;
    // window loss on the device: loss_acc += loss (the micro-batch means, unscaled, as the trainers sum them)
    TRY(mft_add_f32(t->loss_acc, m->loss_dev, t->loss_acc, 1, c.st));
    *stepped = 0;
    if (++t->accum_counter < t->cfg.grad_accum_steps) return MFT_OK;
    t->global_step += 1;
    const float lr = mft_trainer_lr(&t->cfg, t->global_step);
    TRY(mft_model_optimizer_step(m, lr, t->cfg.adam_beta1, t->cfg.adam_beta2, t->cfg.adam_eps, t->cfg.weight_decay, t->cfg.max_grad_norm, 1e-6f));
    float sum = 0.f;
    TRY(mft_memcpy_d2h(&sum, t->loss_acc, 4, c.st));             // the one read-back of the window (synchronises)
    TRY(mft_memset(t->loss_acc, 0, 4, c.st));
    t->accum_counter = 0;
    *stepped = 1;
    if (avg_loss) *avg_loss = sum / static_cast<float>(t->cfg.grad_accum_steps);
    if (lr_used) *lr_used = lr;
    return check_status(m);
}

extern "C" int32_t mft_model_zero_grad(mft_model_t* m) {
    MFT_CHECK_ARG(m, "mft_model_zero_grad: null model");
    if (m->bucket_n == 0) return MFT_OK;
    return mft_memset(m->g_bucket, 0, (size_t)m->bucket_n * 4, m->stream);
}

extern "C" int32_t mft_model_get_final_hidden_host(mft_model_t* m, float* out_host, int64_t n) {
    MFT_CHECK_ARG(m && out_host && n > 0 && n <= m->max_tokens * m->cfg.hidden, "mft_model_get_final_hidden_host: bad argument");
    MFT_CHECK_ARG(n <= m->stage_floats - 64, "mft_model_get_final_hidden_host: too large for the staging buffer");
    TRY(mft_cast_bf16_to_f32(m->hf, m->stage_f32, n, m->stream));
    return mft_memcpy_d2h(out_host, m->stage_f32, (size_t)n * 4, m->stream);
}
