// Step engine: builds the device-resident model (frozen bf16 weights in both
// GEMM layouts, fp32 LoRA buckets, per-layer activation buffers) and runs the
// LoRA fine-tuning step as a fixed sequence of kernels from mft_cuda.h.
// Model construction and parameter upload live in this file; the forward and
// backward schedules are in engine_step.cu.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.cuh"
#include "engine.h"
#include <cstdlib>

using namespace mft;

namespace {

#define TRY(expr)                         \
    do {                                  \
        int32_t s__ = (expr);             \
        if (s__ != MFT_OK) return s__;    \
    } while (0)

template <typename T>
int32_t dalloc(mft_model* m, T** out, int64_t n, bool zero = false, bool activation = false) {
    void* p = nullptr;
    const size_t bytes = (size_t)std::max<int64_t>(n, 1) * sizeof(T);
    TRY(mft_malloc(bytes, m->stream, &p));
    m->allocations.push_back(p);
    if (zero) TRY(mft_memset(p, 0, bytes, m->stream));
    if (activation) m->activation_bytes += (int64_t)bytes;
    *out = static_cast<T*>(p);
    return MFT_OK;
}

int32_t build_group(mft_model* m, LinearGroup& g, int in, const std::vector<int>& outs, const std::vector<bool>& lora,
                    bool with_bias, int rank) {
    g.in = in;
    g.n_total = 0;
    g.slots.clear();
    int panel = 0;
    for (size_t i = 0; i < outs.size(); ++i) {
        LinearSlot s;
        s.in = in; s.out = outs[i]; s.col0 = g.n_total; s.has_lora = lora[i];
        if (s.has_lora) { s.panel_col = panel; panel += rank; g.any_lora = true; }
        g.n_total += outs[i];
        g.slots.push_back(s);
    }
    if (panel > 64) return fail(MFT_ERR_UNSUPPORTED, "LoRA rank x fused linears exceeds the 64-column panel");
    g.k2 = panel;
    TRY(dalloc(m, &g.w_nk, (int64_t)g.n_total * in));
    TRY(dalloc(m, &g.w_kn, (int64_t)in * g.n_total));
    if (with_bias) TRY(dalloc(m, &g.bias, g.n_total, true));
    if (g.any_lora) {
        TRY(dalloc(m, &g.a_nk, (int64_t)64 * in, true));
        TRY(dalloc(m, &g.a_kn, (int64_t)in * 64, true));
        TRY(dalloc(m, &g.b_nk, (int64_t)g.n_total * 64, true));
        TRY(dalloc(m, &g.b_kn, (int64_t)64 * g.n_total, true));
    }
    return MFT_OK;
}

void add_param(mft_model* m, const std::string& name, int64_t rows, int64_t cols, ParamInfo::Kind kind, float* f32_dst = nullptr,
               LinearGroup* g = nullptr, int slot = 0) {
    ParamInfo p;
    p.name = name; p.rows = rows; p.cols = cols; p.kind = kind; p.f32_dst = f32_dst; p.group = g; p.slot = slot;
    m->params.push_back(p);
}

// Registers A and B of one LoRA'd slot in the reference's order and layout.
void add_lora(mft_model* m, LinearSlot& s, int rank, bool peft_layout, bool has_grad) {
    s.lora_idx = (int)m->loras.size();
    LoraInfo a, b;
    if (peft_layout) { a.rows = rank; a.cols = s.in; b.rows = s.out; b.cols = rank; }
    else { a.rows = s.in; a.cols = rank; b.rows = rank; b.cols = s.out; }
    a.has_grad = b.has_grad = has_grad;
    a.offset = m->bucket_n; m->bucket_n += a.rows * a.cols;
    m->bucket_n = (m->bucket_n + 3) / 4 * 4;     // keep every tensor 16-byte aligned
    b.offset = m->bucket_n; m->bucket_n += b.rows * b.cols;
    m->bucket_n = (m->bucket_n + 3) / 4 * 4;
    m->loras.push_back(a);
    m->loras.push_back(b);
}

}  // namespace

extern "C" int32_t mft_model_destroy(mft_model_t* m) {
    if (!m) return MFT_OK;
    cudaStreamSynchronize(m->stream);
    if (m->graph_stream) cudaStreamSynchronize(m->graph_stream);
    for (auto& g : m->graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
    if (m->graph_in) cudaEventDestroy(m->graph_in);
    if (m->graph_out) cudaEventDestroy(m->graph_out);
    if (m->graph_stream) cudaStreamDestroy(m->graph_stream);
    if (m->copy_stream) { cudaStreamSynchronize(m->copy_stream); cudaStreamDestroy(m->copy_stream); }
    for (int i = 0; i < 2; ++i) {
        if (m->slot_ready[i]) cudaEventDestroy(m->slot_ready[i]);
        if (m->slot_free[i]) cudaEventDestroy(m->slot_free[i]);
    }
    for (auto& b : m->merge_backup) { mft_free(b.w_nk, m->stream); mft_free(b.w_kn, m->stream); }
    for (void* p : m->allocations) mft_free(p, m->stream);
    delete m;
    return MFT_OK;
}

extern "C" int32_t mft_model_create(const mft_model_config_t* cfg, mft_stream_t stream, mft_model_t** out) {
    MFT_CHECK_ARG(cfg && out, "mft_model_create: null argument");
    MFT_CHECK_ARG(cfg->family >= 0 && cfg->family <= 2, "mft_model_create: unknown family");
    MFT_CHECK_ARG(cfg->vocab > 0 && cfg->hidden > 0 && cfg->inter > 0 && cfg->layers > 0 && cfg->n_heads > 0 &&
                  cfg->n_kv_heads > 0 && cfg->head_dim > 0 && cfg->max_batch > 0 && cfg->max_seq > 0, "mft_model_create: bad size");
    MFT_CHECK_ARG(cfg->hidden % 8 == 0 && cfg->inter % 8 == 0, "mft_model_create: hidden and inter must be multiples of 8");
    MFT_CHECK_ARG(cfg->n_heads % cfg->n_kv_heads == 0, "mft_model_create: n_heads must be a multiple of n_kv_heads");
    // head sizes 64 / 128 / 256 run on the tiled tensor-core attention kernels, any other even size (test-sized models)
    // on the plain CUDA-core ones; the projections' widths are GEMM row strides and must be multiples of 8 elements
    MFT_CHECK_ARG(cfg->head_dim >= 2 && cfg->head_dim <= 256 && cfg->head_dim % 2 == 0, "mft_model_create: head_dim must be even, at most 256");
    MFT_CHECK_ARG((cfg->n_heads * cfg->head_dim) % 8 == 0 && ((cfg->n_heads + 2 * cfg->n_kv_heads) * cfg->head_dim) % 8 == 0,
                  "mft_model_create: n_heads*head_dim and (n_heads + 2 n_kv_heads)*head_dim must be multiples of 8");
    MFT_CHECK_ARG(cfg->lora_rank >= 0 && cfg->lora_rank <= 64, "mft_model_create: LoRA rank must be at most 64");
    if (!device_status_word()) return fail(MFT_ERR_INVALID_ARG, "mft_model_create: call mft_init first");
    const bool gpt2 = cfg->family == MFT_FAMILY_GPT2, qwen = cfg->family == MFT_FAMILY_QWEN, gemma = cfg->family == MFT_FAMILY_GEMMA;
    MFT_CHECK_ARG(!gpt2 || (cfg->n_heads == cfg->n_kv_heads && cfg->n_heads * cfg->head_dim == cfg->hidden && cfg->n_positions >= cfg->max_seq),
                  "mft_model_create: inconsistent GPT-2 geometry");
    auto* m = new mft_model();
    m->cfg = *cfg;
    m->stream = as_stream(stream);
    m->max_tokens = (int64_t)cfg->max_batch * cfg->max_seq;
    const int H = cfg->hidden, I = cfg->inter, V = cfg->vocab, L = cfg->layers;
    const int nh = cfg->n_heads, nkv = cfg->n_kv_heads, hd = cfg->head_dim, r = cfg->lora_rank;
    const int QD = nh * hd, KD = nkv * hd;
    const uint32_t tg = r > 0 ? cfg->lora_targets : 0;
    const int64_t T = m->max_tokens;
    int32_t st = MFT_OK;
    auto guard = [&](int32_t s) { if (s != MFT_OK && st == MFT_OK) st = s; return s == MFT_OK; };
#define G(expr) if (!guard(expr)) { mft_model_destroy(m); return st; }

    G(dalloc(m, &m->embed, (int64_t)V * H));
    m->ld_t = ((int64_t)V + 63) / 64 * 64;
    G(dalloc(m, &m->embed_t, (int64_t)H * m->ld_t, true));
    G(dalloc(m, &m->final_w, H, true));
    if (gpt2) {
        G(dalloc(m, &m->final_b, H, true));
        G(dalloc(m, &m->pos_embed, (int64_t)cfg->n_positions * H));
    }
    m->layers.resize(L);
    m->bufs.resize(L);

    // ---- frozen parameters in the reference's parameters() order
    if (gpt2) {
        add_param(m, "wte", V, H, ParamInfo::EMBED);
        add_param(m, "wpe", cfg->n_positions, H, ParamInfo::POS_EMBED);
    } else if (qwen) {
        add_param(m, "embed_tokens", V, H, ParamInfo::EMBED);
        add_param(m, "final_norm", 1, H, ParamInfo::NORM, m->final_w);
    } else {
        add_param(m, "embed_tokens", V, H, ParamInfo::EMBED);
        add_param(m, "norm", 1, H, ParamInfo::NORM, m->final_w);
        add_param(m, "lm_head(copy of embed^T)", H, V, ParamInfo::LM_HEAD_COPY);
    }
    for (int l = 0; l < L; ++l) {
        LayerWeights& w = m->layers[l];
        const std::string pre = "layer" + std::to_string(l) + ".";
        G(dalloc(m, &w.ln1_w, H, true));
        G(dalloc(m, &w.ln2_w, H, true));
        if (gpt2) {
            G(dalloc(m, &w.ln1_b, H, true));
            G(dalloc(m, &w.ln2_b, H, true));
            G(build_group(m, w.qkv, H, {3 * H}, {(tg & MFT_LORA_Q) != 0}, true, r));
            G(build_group(m, w.o, H, {H}, {(tg & MFT_LORA_O) != 0}, true, r));
            G(build_group(m, w.gu, H, {I}, {(tg & MFT_LORA_GATE) != 0}, true, r));
            G(build_group(m, w.down, I, {H}, {(tg & MFT_LORA_DOWN) != 0}, true, r));
            add_param(m, pre + "ln_1.weight", 1, H, ParamInfo::NORM, w.ln1_w);
            add_param(m, pre + "ln_1.bias", 1, H, ParamInfo::NORM, w.ln1_b);
            add_param(m, pre + "attn.c_attn.weight", H, 3 * H, ParamInfo::LINEAR, nullptr, &w.qkv, 0);
            add_param(m, pre + "attn.c_attn.bias", 1, 3 * H, ParamInfo::BIAS, nullptr, &w.qkv, 0);
            add_param(m, pre + "attn.c_proj.weight", H, H, ParamInfo::LINEAR, nullptr, &w.o, 0);
            add_param(m, pre + "attn.c_proj.bias", 1, H, ParamInfo::BIAS, nullptr, &w.o, 0);
            add_param(m, pre + "ln_2.weight", 1, H, ParamInfo::NORM, w.ln2_w);
            add_param(m, pre + "ln_2.bias", 1, H, ParamInfo::NORM, w.ln2_b);
            add_param(m, pre + "mlp.c_fc.weight", H, I, ParamInfo::LINEAR, nullptr, &w.gu, 0);
            add_param(m, pre + "mlp.c_fc.bias", 1, I, ParamInfo::BIAS, nullptr, &w.gu, 0);
            add_param(m, pre + "mlp.c_proj.weight", I, H, ParamInfo::LINEAR, nullptr, &w.down, 0);
            add_param(m, pre + "mlp.c_proj.bias", 1, H, ParamInfo::BIAS, nullptr, &w.down, 0);
        } else if (qwen) {
            G(build_group(m, w.qkv, H, {QD, KD, KD}, {(tg & MFT_LORA_Q) != 0, (tg & MFT_LORA_K) != 0, (tg & MFT_LORA_V) != 0}, true, r));
            G(build_group(m, w.o, QD, {H}, {(tg & MFT_LORA_O) != 0}, false, r));
            G(build_group(m, w.gu, H, {I, I}, {false, false}, false, r));
            G(build_group(m, w.down, I, {H}, {false}, false, r));
            add_param(m, pre + "input_layernorm", 1, H, ParamInfo::NORM, w.ln1_w);
            add_param(m, pre + "post_attention_layernorm", 1, H, ParamInfo::NORM, w.ln2_w);
            add_param(m, pre + "q_proj.weight", H, QD, ParamInfo::LINEAR, nullptr, &w.qkv, 0);
            add_param(m, pre + "q_proj.bias", 1, QD, ParamInfo::BIAS, nullptr, &w.qkv, 0);
            add_param(m, pre + "k_proj.weight", H, KD, ParamInfo::LINEAR, nullptr, &w.qkv, 1);
            add_param(m, pre + "k_proj.bias", 1, KD, ParamInfo::BIAS, nullptr, &w.qkv, 1);
            add_param(m, pre + "v_proj.weight", H, KD, ParamInfo::LINEAR, nullptr, &w.qkv, 2);
            add_param(m, pre + "v_proj.bias", 1, KD, ParamInfo::BIAS, nullptr, &w.qkv, 2);
            add_param(m, pre + "o_proj.weight", QD, H, ParamInfo::LINEAR, nullptr, &w.o, 0);
            add_param(m, pre + "gate_proj.weight", H, I, ParamInfo::LINEAR, nullptr, &w.gu, 0);
            add_param(m, pre + "up_proj.weight", H, I, ParamInfo::LINEAR, nullptr, &w.gu, 1);
            add_param(m, pre + "down_proj.weight", I, H, ParamInfo::LINEAR, nullptr, &w.down, 0);
        } else {
            G(dalloc(m, &w.post_attn_w, H, true));
            G(dalloc(m, &w.post_ffn_w, H, true));
            G(dalloc(m, &w.q_norm_w, hd, true));
            G(dalloc(m, &w.k_norm_w, hd, true));
            w.sliding = !(cfg->global_every > 0 && (l + 1) % cfg->global_every == 0);
            G(build_group(m, w.qkv, H, {QD, KD, KD}, {(tg & MFT_LORA_Q) != 0, (tg & MFT_LORA_K) != 0, (tg & MFT_LORA_V) != 0}, false, r));
            G(build_group(m, w.o, QD, {H}, {(tg & MFT_LORA_O) != 0}, false, r));
            G(build_group(m, w.gu, H, {I, I}, {(tg & MFT_LORA_GATE) != 0, (tg & MFT_LORA_UP) != 0}, false, r));
            G(build_group(m, w.down, I, {H}, {(tg & MFT_LORA_DOWN) != 0}, false, r));
            add_param(m, pre + "input_layernorm", 1, H, ParamInfo::NORM, w.ln1_w);
            add_param(m, pre + "post_attention_layernorm", 1, H, ParamInfo::NORM, w.post_attn_w);
            add_param(m, pre + "pre_feedforward_layernorm", 1, H, ParamInfo::NORM, w.ln2_w);
            add_param(m, pre + "post_feedforward_layernorm", 1, H, ParamInfo::NORM, w.post_ffn_w);
            add_param(m, pre + "q_proj.weight", H, QD, ParamInfo::LINEAR, nullptr, &w.qkv, 0);
            add_param(m, pre + "k_proj.weight", H, KD, ParamInfo::LINEAR, nullptr, &w.qkv, 1);
            add_param(m, pre + "v_proj.weight", H, KD, ParamInfo::LINEAR, nullptr, &w.qkv, 2);
            add_param(m, pre + "o_proj.weight", QD, H, ParamInfo::LINEAR, nullptr, &w.o, 0);
            add_param(m, pre + "q_norm", 1, hd, ParamInfo::NORM, w.q_norm_w);
            add_param(m, pre + "k_norm", 1, hd, ParamInfo::NORM, w.k_norm_w);
            add_param(m, pre + "gate_proj.weight", H, I, ParamInfo::LINEAR, nullptr, &w.gu, 0);
            add_param(m, pre + "up_proj.weight", H, I, ParamInfo::LINEAR, nullptr, &w.gu, 1);
            add_param(m, pre + "down_proj.weight", I, H, ParamInfo::LINEAR, nullptr, &w.down, 0);
        }
    }
    if (gpt2) {
        add_param(m, "ln_f.weight", 1, H, ParamInfo::NORM, m->final_w);
        add_param(m, "ln_f.bias", 1, H, ParamInfo::NORM, m->final_b);
    }

    // ---- LoRA tensors in get_lora_parameters() order
    for (int l = 0; l < L; ++l) {
        LayerWeights& w = m->layers[l];
        auto reg = [&](LinearSlot& s, bool has_grad) { if (s.has_lora) add_lora(m, s, r, gemma, has_grad); };
        if (gpt2) {
            reg(w.qkv.slots[0], cfg->gpt2_detach_attn == 0);   // the reference severs autograd at the QKV split
            reg(w.o.slots[0], true); reg(w.gu.slots[0], true); reg(w.down.slots[0], true);
        } else if (qwen) {
            reg(w.qkv.slots[0], true); reg(w.qkv.slots[2], true); reg(w.qkv.slots[1], true); reg(w.o.slots[0], true);   // q, v, k, o
        } else {
            reg(w.qkv.slots[0], true); reg(w.qkv.slots[1], true); reg(w.qkv.slots[2], true); reg(w.o.slots[0], true);
            reg(w.gu.slots[0], true); reg(w.gu.slots[1], true); reg(w.down.slots[0], true);
        }
    }
    if (m->bucket_n > 0) {
        G(dalloc(m, &m->p_bucket, m->bucket_n, true));
        G(dalloc(m, &m->g_bucket, m->bucket_n, true));
        G(dalloc(m, &m->m_bucket, m->bucket_n, true));
        G(dalloc(m, &m->v_bucket, m->bucket_n, true));
    }
    G(dalloc(m, &m->sqnorm, 4, true));

    // ---- gradient panels (one allocation) and the pack / unpack tables
    {
        int64_t total = 0;
        for (auto& w : m->layers)
            for (LinearGroup* g : {&w.qkv, &w.o, &w.gu, &w.down})
                if (g->any_lora) total += (int64_t)g->in * 64 + (int64_t)64 * g->n_total;
        m->grad_pan_floats = total;
        if (total > 0) G(dalloc(m, &m->grad_pan_base, total, true));
        int64_t off = 0;
        std::vector<mft_block_copy_t> pack, unpack;
        for (auto& w : m->layers)
            for (LinearGroup* g : {&w.qkv, &w.o, &w.gu, &w.down}) {
                if (!g->any_lora) continue;
                g->da_pan = m->grad_pan_base + off; off += (int64_t)g->in * 64;
                g->db_pan = m->grad_pan_base + off; off += (int64_t)64 * g->n_total;
                for (auto& s : g->slots) {
                    if (!s.has_lora) continue;
                    const LoraInfo& A = m->loras[s.lora_idx];
                    const LoraInfo& B = m->loras[s.lora_idx + 1];
                    float* pa = m->p_bucket + A.offset; float* pb = m->p_bucket + B.offset;
                    float* ga = m->g_bucket + A.offset; float* gb = m->g_bucket + B.offset;
                    const int pc = s.panel_col;
                    auto E = [](const void* src, void* dst, int rows, int cols, int sld, int dld, int tr) {
                        mft_block_copy_t e; e.src = src; e.dst = dst; e.rows = rows; e.cols = cols; e.src_ld = sld; e.dst_ld = dld; e.transpose = tr; e.pad = 0; return e;
                    };
                    if (gemma) {   // A [r,in], B [out,r]
                        pack.push_back(E(pa, g->a_nk + (int64_t)pc * g->in, r, s.in, s.in, g->in, 0));
                        pack.push_back(E(pa, g->a_kn + pc, r, s.in, s.in, 64, 1));
                        pack.push_back(E(pb, g->b_nk + (int64_t)s.col0 * 64 + pc, s.out, r, r, 64, 0));
                        pack.push_back(E(pb, g->b_kn + (int64_t)pc * g->n_total + s.col0, s.out, r, r, g->n_total, 1));
                        if (A.has_grad) {
                            unpack.push_back(E(g->da_pan + pc, ga, s.in, r, 64, s.in, 1));                                  // [in,r] block -> [r,in]
                            unpack.push_back(E(g->db_pan + (int64_t)pc * g->n_total + s.col0, gb, r, s.out, g->n_total, r, 1));  // [r,out] block -> [out,r]
                        }
                    } else {       // A [in,r], B [r,out]
                        pack.push_back(E(pa, g->a_nk + (int64_t)pc * g->in, s.in, r, r, g->in, 1));
                        pack.push_back(E(pa, g->a_kn + pc, s.in, r, r, 64, 0));
                        pack.push_back(E(pb, g->b_nk + (int64_t)s.col0 * 64 + pc, r, s.out, s.out, 64, 1));
                        pack.push_back(E(pb, g->b_kn + (int64_t)pc * g->n_total + s.col0, r, s.out, s.out, g->n_total, 0));
                        if (A.has_grad) {
                            unpack.push_back(E(g->da_pan + pc, ga, s.in, r, 64, r, 0));
                            unpack.push_back(E(g->db_pan + (int64_t)pc * g->n_total + s.col0, gb, r, s.out, g->n_total, s.out, 0));
                        }
                    }
                }
            }
        m->n_pack = (int)pack.size(); m->n_unpack = (int)unpack.size();
        if (m->n_pack) {
            G(dalloc(m, &m->pack_table, m->n_pack));
            G(mft_memcpy_h2d(m->pack_table, pack.data(), pack.size() * sizeof(mft_block_copy_t), m->stream));
        }
        if (m->n_unpack) {
            G(dalloc(m, &m->unpack_table, m->n_unpack));
            G(mft_memcpy_h2d(m->unpack_table, unpack.data(), unpack.size() * sizeof(mft_block_copy_t), m->stream));
        }
        G(check_cuda(cudaStreamSynchronize(m->stream), "table upload"));   // the host vectors go out of scope
    }

    // ---- RoPE tables (host expression identical to the reference's)
    if (!gpt2) {
        const int64_t n = (int64_t)cfg->max_seq * (hd / 2);
        std::vector<float> c(n), s(n);
        G(dalloc(m, &m->cos_g, n)); G(dalloc(m, &m->sin_g, n));
        G(mft_rope_table_host(c.data(), s.data(), cfg->max_seq, hd, cfg->rope_theta));
        G(mft_memcpy_h2d(m->cos_g, c.data(), n * 4, m->stream)); G(mft_memcpy_h2d(m->sin_g, s.data(), n * 4, m->stream));
        G(check_cuda(cudaStreamSynchronize(m->stream), "rope upload"));
        if (gemma) {
            G(dalloc(m, &m->cos_l, n)); G(dalloc(m, &m->sin_l, n));
            G(mft_rope_table_host(c.data(), s.data(), cfg->max_seq, hd, cfg->rope_local_theta));
            G(mft_memcpy_h2d(m->cos_l, c.data(), n * 4, m->stream)); G(mft_memcpy_h2d(m->sin_l, s.data(), n * 4, m->stream));
            G(check_cuda(cudaStreamSynchronize(m->stream), "rope upload"));
        }
    }

    // ---- activations
    const int64_t QKV = QD + 2 * KD, GU = gpt2 ? I : 2 * I;
    for (int l = 0; l < L; ++l) {
        LayerBuffers& b = m->bufs[l];
        LayerWeights& w = m->layers[l];
        G(dalloc(m, &b.x, T * H, false, true));
        G(dalloc(m, &b.h1, T * H, false, true));
        G(dalloc(m, &b.rstd1, T, false, true));
        if (gpt2) { G(dalloc(m, &b.mean1, T, false, true)); G(dalloc(m, &b.mean3, T, false, true)); }
        G(dalloc(m, &b.qkv, T * QKV, false, true));
        if (!gpt2) G(dalloc(m, &b.qk_r, T * (QD + KD), false, true));
        if (gemma) { G(dalloc(m, &b.rstd_q, T * nh, false, true)); G(dalloc(m, &b.rstd_k, T * nkv, false, true)); }
        G(dalloc(m, &b.o, T * QD, false, true));
        G(dalloc(m, &b.lse, T * nh, false, true));
        G(dalloc(m, &b.attn_out, T * H, false, true));
        G(dalloc(m, &b.x_mid, T * H, false, true));
        G(dalloc(m, &b.h2, T * H, false, true));
        G(dalloc(m, &b.rstd3, T, false, true));
        G(dalloc(m, &b.gu, T * GU, false, true));
        G(dalloc(m, &b.act, T * I, false, true));
        G(dalloc(m, &b.mlp_out, T * H, false, true));
        if (gemma) { G(dalloc(m, &b.rstd2, T, false, true)); G(dalloc(m, &b.rstd4, T, false, true)); }
        if (w.qkv.any_lora) G(dalloc(m, &b.xa_qkv, T * 64, false, true));
        if (w.o.any_lora) G(dalloc(m, &b.xa_o, T * 64, false, true));
        if (w.gu.any_lora) G(dalloc(m, &b.xa_gu, T * 64, false, true));
        if (w.down.any_lora) G(dalloc(m, &b.xa_d, T * 64, false, true));
    }
    G(dalloc(m, &m->ids, T)); G(dalloc(m, &m->labels, T));
    G(dalloc(m, &m->x_final, T * H, false, true));
    G(dalloc(m, &m->hf, T * H, false, true));
    G(dalloc(m, &m->rstd_f, T)); G(dalloc(m, &m->mean_f, T));
    G(dalloc(m, &m->dx, T * H, false, true));
    G(dalloc(m, &m->t_h, T * H, false, true));
    G(dalloc(m, &m->t_i, T * I, false, true));
    G(dalloc(m, &m->t_gu, T * GU, false, true));
    G(dalloc(m, &m->t_o, T * QD, false, true));
    G(dalloc(m, &m->t_qk, T * (QD + KD), false, true));
    G(dalloc(m, &m->t_qkv, T * QKV, false, true));
    G(dalloc(m, &m->t_pan, T * 64, false, true));
    G(dalloc(m, &m->attn_delta, T * nh, false, true));
    if (nh > nkv) G(dalloc(m, &m->attn_dkv_acc, 2 * T * nkv * hd, false, true));
    G(dalloc(m, &m->loss_dev, 4, true)); G(dalloc(m, &m->n_valid_dev, 4, true)); G(dalloc(m, &m->status_dev, 4, true));
    G(dalloc(m, &m->ce_lse, T));
    m->ce_ws_bytes = mft_lmhead_ce_workspace_bytes(T, H, V);
    if (const char* e = std::getenv("MFT_CE_ONEPASS")) m->ce_onepass = std::atoi(e) != 0;
    if (const char* e = std::getenv("MFT_STEP_GRAPH")) m->use_graph = std::atoi(e) != 0;
    if (const char* e = std::getenv("MFT_FUSE_GLU")) { m->fuse_glu = std::atoi(e) != 0; m->fuse_glu_fwd = std::atoi(e) >= 2; }
    if (const char* e = std::getenv("MFT_FUSE_NORMS")) m->fuse_norms = std::atoi(e) != 0;
    { uint8_t* ws = nullptr; G(dalloc(m, &ws, m->ce_ws_bytes, false, true)); m->ce_ws = ws; }
    m->stage_floats = 32ll << 20;
    G(dalloc(m, &m->stage_f32, m->stage_floats));
    G(check_cuda(cudaStreamSynchronize(m->stream), "model create"));
#undef G
    *out = m;
    return MFT_OK;
}

// ---------------------------------------------------------------- parameter access
extern "C" int32_t mft_model_param_count(const mft_model_t* m) { return m ? (int32_t)m->params.size() : 0; }
extern "C" int32_t mft_model_param_shape(const mft_model_t* m, int32_t idx, int64_t* rows, int64_t* cols) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->params.size() && rows && cols, "mft_model_param_shape: bad argument");
    *rows = m->params[idx].rows; *cols = m->params[idx].cols;
    return MFT_OK;
}

namespace {
// Installs rows [r0, r0+nr) of parameter `p` from a device f32 buffer holding exactly those rows.
int32_t install_rows(mft_model* m, const ParamInfo& p, const float* src_dev, int64_t r0, int64_t nr) {
    mft_stream_t st = m->stream;
    switch (p.kind) {
        case ParamInfo::EMBED:
            return mft_cast_f32_to_bf16(src_dev, m->embed + r0 * p.cols, nr * p.cols, st);
        case ParamInfo::POS_EMBED:
            return mft_cast_f32_to_bf16(src_dev, m->pos_embed + r0 * p.cols, nr * p.cols, st);
        case ParamInfo::LM_HEAD_COPY:
            return MFT_OK;   // the device keeps a single table; its transpose is derived from the embedding
        case ParamInfo::NORM:
            return mft_memcpy_d2d(p.f32_dst, src_dev, p.cols * 4, st);
        case ParamInfo::BIAS: {
            const LinearSlot& s = p.group->slots[p.slot];
            return mft_memcpy_d2d(p.group->bias + s.col0, src_dev, p.cols * 4, st);
        }
        case ParamInfo::LINEAR: {
            // host layout [in, out]; whole matrix at once (r0 == 0, nr == in)
            LinearGroup* g = p.group;
            const LinearSlot& s = g->slots[p.slot];
            TRY(mft_transpose_f32_to_bf16(src_dev, g->w_nk + (int64_t)s.col0 * g->in, s.in, s.out, st));
            mft_block_copy_t e; e.src = src_dev; e.dst = g->w_kn + s.col0; e.rows = s.in; e.cols = s.out; e.src_ld = s.out; e.dst_ld = g->n_total; e.transpose = 0; e.pad = 0;
            // one-entry copy table, parked in the last 256 bytes of the staging buffer
            mft_block_copy_t* tbl = reinterpret_cast<mft_block_copy_t*>(m->stage_f32 + m->stage_floats - 64);
            TRY(mft_memcpy_h2d(tbl, &e, sizeof(e), st));
            TRY(check_cuda(cudaStreamSynchronize(m->stream), "table upload"));
            return mft_pack_blocks_bf16(tbl, 1, st);
        }
    }
    return MFT_OK;
}

int32_t finish_param(mft_model* m, const ParamInfo& p) {
    if (p.kind == ParamInfo::EMBED)
        return mft_transpose_bf16_ld(m->embed, m->embed_t, p.rows, p.cols, m->ld_t, m->stream);
    return MFT_OK;
}
}  // namespace

extern "C" int32_t mft_model_set_param_dev(mft_model_t* m, int32_t idx, const float* data_dev) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->params.size() && data_dev, "mft_model_set_param_dev: bad argument");
    const ParamInfo& p = m->params[idx];
    TRY(install_rows(m, p, data_dev, 0, p.rows));
    return finish_param(m, p);
}

extern "C" int32_t mft_model_set_param_host(mft_model_t* m, int32_t idx, const float* data_host) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->params.size() && data_host, "mft_model_set_param_host: bad argument");
    const ParamInfo& p = m->params[idx];
    if (p.kind == ParamInfo::LM_HEAD_COPY) return MFT_OK;
    const int64_t usable = m->stage_floats - 64;
    if (p.kind == ParamInfo::LINEAR) {
        MFT_CHECK_ARG(p.rows * p.cols <= usable, "mft_model_set_param_host: linear larger than the staging buffer");
        TRY(mft_memcpy_h2d(m->stage_f32, data_host, (size_t)p.rows * p.cols * 4, m->stream));
        TRY(install_rows(m, p, m->stage_f32, 0, p.rows));
        return check_cuda(cudaStreamSynchronize(m->stream), "param upload");
    }
    const int64_t rows_per = std::max<int64_t>(1, usable / p.cols);
    for (int64_t r0 = 0; r0 < p.rows; r0 += rows_per) {
        const int64_t nr = std::min(rows_per, p.rows - r0);
        TRY(mft_memcpy_h2d(m->stage_f32, data_host + r0 * p.cols, (size_t)nr * p.cols * 4, m->stream));
        TRY(install_rows(m, p, m->stage_f32, r0, nr));
        TRY(check_cuda(cudaStreamSynchronize(m->stream), "param upload"));
    }
    TRY(finish_param(m, p));
    return check_cuda(cudaStreamSynchronize(m->stream), "param upload");
}

// bf16 source: the bits are the ones the device stores, so they go up as they are (half the bytes of the f32 path,
// no conversion loop on the host) and are placed by device copies / transposes.
extern "C" int32_t mft_model_set_param_host_bf16(mft_model_t* m, int32_t idx, const void* data_bf16_host, int32_t stored_transposed) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->params.size() && data_bf16_host, "mft_model_set_param_host_bf16: bad argument");
    const ParamInfo& p = m->params[idx];
    const uint16_t* src = static_cast<const uint16_t*>(data_bf16_host);
    const int64_t n = p.rows * p.cols;
    MFT_CHECK_ARG(!stored_transposed || p.kind == ParamInfo::LINEAR, "mft_model_set_param_host_bf16: only linear weights come transposed");
    auto sync = [&] { return check_cuda(cudaStreamSynchronize(m->stream), "param upload"); };
    switch (p.kind) {
        case ParamInfo::LM_HEAD_COPY:
            return MFT_OK;
        case ParamInfo::EMBED:
        case ParamInfo::POS_EMBED: {        // straight into the table
            __nv_bfloat16* dst = p.kind == ParamInfo::EMBED ? m->embed : m->pos_embed;
            TRY(mft_memcpy_h2d(dst, src, (size_t)n * 2, m->stream));
            TRY(finish_param(m, p));
            return sync();
        }
        case ParamInfo::LINEAR: {
            LinearGroup* g = p.group;
            const LinearSlot& s = g->slots[p.slot];
            const int64_t stage_bytes = (m->stage_floats - 64) * 4;
            if (stored_transposed) {
                // [out, in] as stored IS this slot's rows of w_nk; w_kn gets the transpose
                __nv_bfloat16* nk = g->w_nk + (int64_t)s.col0 * g->in;
                TRY(mft_memcpy_h2d(nk, src, (size_t)n * 2, m->stream));
                TRY(mft_transpose_bf16_ld(nk, g->w_kn + s.col0, s.out, s.in, g->n_total, m->stream));
                return sync();
            }
            if (n * 6 > stage_bytes) return fail(MFT_ERR_UNSUPPORTED, "mft_model_set_param_host_bf16: linear larger than the staging buffer");
            break;                          // [in, out]: through the f32 staging path below
        }
        default:
            MFT_CHECK_ARG(n * 6 <= (m->stage_floats - 64) * 4, "mft_model_set_param_host_bf16: tensor larger than the staging buffer");
            break;
    }
    // raw bits behind the f32 staging area, widened on the device (exact), then the usual placement
    void* raw = reinterpret_cast<uint8_t*>(m->stage_f32) + (size_t)((n * 4 + 255) / 256 * 256);
    TRY(mft_memcpy_h2d(raw, src, (size_t)n * 2, m->stream));
    TRY(mft_cast_bf16_to_f32(raw, m->stage_f32, n, m->stream));
    TRY(install_rows(m, p, m->stage_f32, 0, p.rows));
    TRY(finish_param(m, p));
    return sync();
}

extern "C" int32_t mft_model_lora_count(const mft_model_t* m) { return m ? (int32_t)m->loras.size() : 0; }
extern "C" int32_t mft_model_lora_shape(const mft_model_t* m, int32_t idx, int64_t* rows, int64_t* cols) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->loras.size() && rows && cols, "mft_model_lora_shape: bad argument");
    *rows = m->loras[idx].rows; *cols = m->loras[idx].cols;
    return MFT_OK;
}
extern "C" int32_t mft_model_lora_has_grad(const mft_model_t* m, int32_t idx) {
    return (m && idx >= 0 && idx < (int)m->loras.size() && m->loras[idx].has_grad) ? 1 : 0;
}
extern "C" int32_t mft_model_set_lora_host(mft_model_t* m, int32_t idx, const float* data_host) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->loras.size() && data_host, "mft_model_set_lora_host: bad argument");
    MFT_CHECK_ARG(!m->merged, "mft_model_set_lora_host: the adapters are merged into the base weights: unmerge first");
    const LoraInfo& t = m->loras[idx];
    TRY(mft_memcpy_h2d(m->p_bucket + t.offset, data_host, (size_t)t.rows * t.cols * 4, m->stream));
    m->panels_dirty = true;
    return check_cuda(cudaStreamSynchronize(m->stream), "lora upload");
}
extern "C" int32_t mft_model_get_lora_host(mft_model_t* m, int32_t idx, float* data_host) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->loras.size() && data_host, "mft_model_get_lora_host: bad argument");
    const LoraInfo& t = m->loras[idx];
    return mft_memcpy_d2h(data_host, m->p_bucket + t.offset, (size_t)t.rows * t.cols * 4, m->stream);
}
extern "C" int32_t mft_model_get_lora_grad_host(mft_model_t* m, int32_t idx, float* data_host) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->loras.size() && data_host, "mft_model_get_lora_grad_host: bad argument");
    const LoraInfo& t = m->loras[idx];
    return mft_memcpy_d2h(data_host, m->g_bucket + t.offset, (size_t)t.rows * t.cols * 4, m->stream);
}
extern "C" int32_t mft_model_lora_offset(const mft_model_t* m, int32_t idx, int64_t* offset) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->loras.size() && offset, "mft_model_lora_offset: bad argument");
    *offset = m->loras[idx].offset;
    return MFT_OK;
}
extern "C" int32_t mft_model_mark_lora_dirty(mft_model_t* m) {
    MFT_CHECK_ARG(m, "mft_model_mark_lora_dirty: null model");
    MFT_CHECK_ARG(!m->merged, "mft_model_mark_lora_dirty: the adapters are merged into the base weights: unmerge first");
    m->panels_dirty = true;
    return MFT_OK;
}
extern "C" int32_t mft_model_buckets(mft_model_t* m, float** params_dev, float** grads_dev, int64_t* n) {
    MFT_CHECK_ARG(m, "mft_model_buckets: null model");
    if (params_dev) *params_dev = m->p_bucket;
    if (grads_dev) *grads_dev = m->g_bucket;
    if (n) *n = m->bucket_n;
    return MFT_OK;
}
// ---------------------------------------------------------------- merge / unmerge of the adapters
// LoRALinear::merge_to_base (nn/lora_linear.cpp:470-483, apply_lora_delta_to_base :107-139): for every adapted slice
//   W[i, col0 + o] <- W[i, col0 + o] + scale * float( sum_r double(A[i,r]) * double(B[r,o]) ),
// written back in the weight's storage type (bf16 here); both device layouts of the weight get the same value.
// unmerge_from_base (:485-508) restores the saved bytes.
namespace {
__global__ void lora_merge_kernel(const float* __restrict__ A, const float* __restrict__ B, int a_is_r_by_in, int in, int out, int r,
                                  float scale, mft::bf16* __restrict__ w_nk, mft::bf16* __restrict__ w_kn, int n_total, int col0) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)in * out) return;
    const int i = (int)(idx / out), o = (int)(idx % out);
    double delta = 0.0;
    for (int k = 0; k < r; ++k) {
        const float a = a_is_r_by_in ? A[(int64_t)k * in + i] : A[(int64_t)i * r + k];      // Gemma keeps A [r,in], B [out,r]
        const float b = a_is_r_by_in ? B[(int64_t)o * r + k] : B[(int64_t)k * out + o];
        delta += (double)a * (double)b;
    }
    const int64_t kn = (int64_t)i * n_total + col0 + o;
    const float updated = __fadd_rn(__bfloat162float(w_kn[kn]), __fmul_rn(scale, (float)delta));
    const mft::bf16 v = __float2bfloat16_rn(updated);
    w_kn[kn] = v;
    w_nk[(int64_t)(col0 + o) * in + i] = v;
}
}  // namespace

extern "C" int32_t mft_model_merge_lora(mft_model_t* m) {
    MFT_CHECK_ARG(m, "mft_model_merge_lora: null model");
    if (m->merged || m->cfg.lora_rank <= 0) return MFT_OK;
    const bool gemma = m->cfg.family == MFT_FAMILY_GEMMA;
    const int r = m->cfg.lora_rank;
    const float scale = m->cfg.lora_alpha / (float)r;
    for (auto& w : m->layers)
        for (LinearGroup* g : {&w.qkv, &w.o, &w.gu, &w.down}) {
            if (!g->any_lora) continue;
            const size_t bytes = (size_t)g->in * g->n_total * sizeof(bf16);
            void *b1 = nullptr, *b2 = nullptr;
            int32_t s = mft_malloc(bytes, m->stream, &b1);
            if (s == MFT_OK) s = mft_malloc(bytes, m->stream, &b2);
            if (s == MFT_OK) s = mft_memcpy_d2d(b1, g->w_nk, bytes, m->stream);
            if (s == MFT_OK) s = mft_memcpy_d2d(b2, g->w_kn, bytes, m->stream);
            if (s != MFT_OK) {
                if (b1) mft_free(b1, m->stream);
                if (b2) mft_free(b2, m->stream);
                m->merged = true;                  // so that the partial merge is rolled back
                mft_model_unmerge_lora(m);
                return s;
            }
            m->merge_backup.push_back({g, static_cast<bf16*>(b1), static_cast<bf16*>(b2)});
            for (auto& sl : g->slots) {
                if (!sl.has_lora) continue;
                const float* A = m->p_bucket + m->loras[sl.lora_idx].offset;
                const float* B = m->p_bucket + m->loras[sl.lora_idx + 1].offset;
                const int64_t n = (int64_t)sl.in * sl.out;
                lora_merge_kernel<<<(unsigned)((n + 255) / 256), 256, 0, m->stream>>>(A, B, gemma ? 1 : 0, sl.in, sl.out, r, scale, g->w_nk, g->w_kn,
                                                                                      g->n_total, sl.col0);
                MFT_LAUNCH_CHECK("lora_merge");
            }
        }
    m->merged = true;
    return MFT_OK;
}

extern "C" int32_t mft_model_unmerge_lora(mft_model_t* m) {
    MFT_CHECK_ARG(m, "mft_model_unmerge_lora: null model");
    if (!m->merged) return MFT_OK;
    int32_t first = MFT_OK;
    for (auto& b : m->merge_backup) {
        const size_t bytes = (size_t)b.group->in * b.group->n_total * sizeof(bf16);
        int32_t s = mft_memcpy_d2d(b.group->w_nk, b.w_nk, bytes, m->stream);
        if (s == MFT_OK) s = mft_memcpy_d2d(b.group->w_kn, b.w_kn, bytes, m->stream);
        if (s != MFT_OK && first == MFT_OK) first = s;
    }
    if (int32_t s = check_cuda(cudaStreamSynchronize(m->stream), "unmerge sync")) { if (first == MFT_OK) first = s; }
    for (auto& b : m->merge_backup) { mft_free(b.w_nk, m->stream); mft_free(b.w_kn, m->stream); }
    m->merge_backup.clear();
    m->merged = false;
    return first;
}

extern "C" int32_t mft_model_is_merged(const mft_model_t* m) { return m && m->merged ? 1 : 0; }

extern "C" int64_t mft_model_activation_bytes(const mft_model_t* m) { return m ? m->activation_bytes : 0; }
