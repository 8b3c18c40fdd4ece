"""Test infrastructure: CPU restatement (numpy) of the reference's arithmetic for the
LoRA fine-tuning step, operator by operator.

Each function follows the cited reference code (paths relative to
operator/finetune_ops/).  It is pinned against outputs of the compiled
reference itself (tests/golden/*.npz, produced by tests/golden/make_golden.py
through oracle/_ref/ref_driver_*) in the CPU test-suite.  Only tests/, the
smoke check and bench.py's CPU-baseline leg may import this module: it is the
checker, never the product path.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32
MASK_VALUE = f32(-1e10)   # core/ops.cpp:2174, graph/gemma_model.cpp:175


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 -> fp32 (core/dtype.h:114-121)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + bias) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


# ---------------------------------------------------------------- matmul / LoRA linear
def matmul(a, b):
    """ops::matmul core/ops.cpp:619-822 (fp32, accumulation order free)."""
    return (a.astype(np.float64) @ b.astype(np.float64)).astype(f32)


def lora_linear_fwd(x, W, bias, A, B, scale):
    """LoRALinear::forward nn/lora_linear.cpp:336-468: y = xW (+b) + scale*((xA)B); A [in,r], B [r,out]."""
    x2 = x.reshape(-1, x.shape[-1]).astype(np.float64)
    y = x2 @ W.astype(np.float64)
    if bias is not None:
        y = y + bias.astype(np.float64)
    y = y + scale * ((x2 @ A.astype(np.float64)) @ B.astype(np.float64))
    return y.astype(f32).reshape(*x.shape[:-1], W.shape[1])


def lora_linear_bwd(x, W, A, B, scale, dy):
    """Generic autograd of the chain above (MatmulBackward core/backward_functions.cpp:94-147)."""
    x2 = x.reshape(-1, x.shape[-1]).astype(np.float64)
    g = dy.reshape(-1, dy.shape[-1]).astype(np.float64)
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    gB = g @ B64.T                       # [T, r]
    dx = g @ W.astype(np.float64).T + scale * (gB @ A64.T)
    dA = scale * (x2.T @ gB)
    dB = scale * ((x2 @ A64).T @ g)
    return dx.astype(f32).reshape(x.shape), dA.astype(f32), dB.astype(f32)


# ---------------------------------------------------------------- attention chain
def repeat_kv(kv, rep):
    """ops::repeat_kv_heads core/ops.cpp:2260-2335: out[b, h*rep + r] = kv[b, h]."""
    return np.repeat(kv, rep, axis=1)


def repeat_kv_bwd(dout, rep):
    """RepeatKVHeadsBackward core/backward_functions.cpp:693-726: sum over the rep copies."""
    b, nh, s, d = dout.shape
    return dout.reshape(b, nh // rep, rep, s, d).sum(axis=2).astype(f32)


def rope_tables(seq, hd, theta):
    """apply_rope core/ops.cpp:2364-2372: freq = 1/powf(theta, 2d/hd), angle = pos*freq, all fp32."""
    d = np.arange(hd // 2, dtype=f32)
    freq = (f32(1.0) / np.power(f32(theta), f32(2.0) * d / f32(hd), dtype=f32)).astype(f32)
    ang = (np.arange(seq, dtype=f32)[:, None] * freq[None, :]).astype(f32)
    return np.cos(ang).astype(f32), np.sin(ang).astype(f32)


def rope_fwd(x, theta):
    """Rotate-half pairing (d, d + hd/2), core/ops.cpp:2337-2414; x [B,H,S,hd]."""
    s, hd = x.shape[2], x.shape[3]
    c, sn = rope_tables(s, hd, theta)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return np.concatenate([x1 * c - x2 * sn, x1 * sn + x2 * c], axis=-1).astype(f32)


def rope_bwd(dy, theta):
    """ApplyRoPEBackward core/backward_functions.cpp:728-774 (the transposed rotation)."""
    s, hd = dy.shape[2], dy.shape[3]
    c, sn = rope_tables(s, hd, theta)
    g1, g2 = dy[..., : hd // 2], dy[..., hd // 2:]
    return np.concatenate([g1 * c + g2 * sn, -g1 * sn + g2 * c], axis=-1).astype(f32)


def additive_mask(seq, window=0):
    """create_causal_mask core/ops.cpp:2167-2180; GemmaModel::build_sliding_mask graph/gemma_model.cpp:272-285."""
    i = np.arange(seq)[:, None]
    j = np.arange(seq)[None, :]
    ok = (j <= i) & ((window <= 0) | (i - j < window))
    return np.where(ok, f32(0), MASK_VALUE).astype(f32)


def attention_fwd_bwd(q, k, v, dO, scale, window=0, rope_theta=0.0):
    """repeat_kv -> transpose -> matmul -> mul(scale) -> add(mask) -> softmax -> matmul and its
    autograd (graph/gemma_model.cpp:487-505; softmax core/ops.cpp:1307-1363; SoftmaxBackward
    core/backward_functions.cpp:306-349).  q [B,nh,S,hd]; k,v [B,nkv,S,hd].  float64 inside."""
    nh, nkv = q.shape[1], k.shape[1]
    rep = nh // nkv
    qq = rope_fwd(q, rope_theta) if rope_theta > 0 else q
    kk = rope_fwd(k, rope_theta) if rope_theta > 0 else k
    kf = repeat_kv(kk, rep).astype(np.float64)
    vf = repeat_kv(v, rep).astype(np.float64)
    q64 = qq.astype(np.float64)
    scores = np.einsum("bhid,bhjd->bhij", q64, kf) * scale + additive_mask(q.shape[2], window).astype(np.float64)
    scores -= scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    out = np.einsum("bhij,bhjd->bhid", p, vf)
    g = dO.astype(np.float64)
    dvf = np.einsum("bhij,bhid->bhjd", p, g)
    dp = np.einsum("bhid,bhjd->bhij", g, vf)
    ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True)) * scale
    dq = np.einsum("bhij,bhjd->bhid", ds, kf)
    dkf = np.einsum("bhij,bhid->bhjd", ds, q64)
    dk = repeat_kv_bwd(dkf, rep)
    dv = repeat_kv_bwd(dvf, rep)
    dq = dq.astype(f32)
    if rope_theta > 0:
        dq, dk = rope_bwd(dq, rope_theta), rope_bwd(dk, rope_theta)
    return out.astype(f32), dq, dk.astype(f32), dv.astype(f32)


# ---------------------------------------------------------------- norms
def rms_norm_fwd(x, w, eps, unit_offset):
    """rms_norm (1+w) core/ops.cpp:1677-1725 / rms_norm_affine (w) :1728-1762; double sum of squares."""
    x64 = x.astype(np.float64)
    inv = 1.0 / np.sqrt((x64 * x64).mean(axis=-1, keepdims=True) + float(eps))
    scale = (1.0 + w.astype(np.float64)) if unit_offset else w.astype(np.float64)
    return (x64 * inv * scale).astype(f32)


def rms_norm_bwd(dy, x, w, eps, unit_offset):
    """RMSNormBackward core/backward_functions.cpp:492-532 (and :534-570 for the affine form)."""
    x64, g64 = x.astype(np.float64), dy.astype(np.float64)
    d = x.shape[-1]
    inv = 1.0 / np.sqrt((x64 * x64).mean(axis=-1, keepdims=True) + float(eps))
    scale = (1.0 + w.astype(np.float64)) if unit_offset else w.astype(np.float64)
    gw = g64 * scale
    dot = (gw * x64).sum(axis=-1, keepdims=True)
    dx = gw * inv - x64 * (inv ** 3) / d * dot
    dw = (g64 * x64 * inv).reshape(-1, d).sum(axis=0)
    return dx.astype(f32), dw.astype(f32)


def layer_norm_fwd(x, w, b, eps):
    """layer_norm core/ops.cpp:1592-1646 (biased variance)."""
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=-1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=-1, keepdims=True)
    return ((x64 - mean) / np.sqrt(var + float(eps)) * w + b).astype(f32)


def layer_norm_bwd(dy, x, w, eps):
    """LayerNormBackward core/backward_functions.cpp:434-490."""
    x64, g64 = x.astype(np.float64), dy.astype(np.float64)
    d = x.shape[-1]
    mean = x64.mean(axis=-1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(var + float(eps))
    xh = (x64 - mean) * inv
    gw = g64 * w.astype(np.float64)
    dx = inv / d * (d * gw - gw.sum(axis=-1, keepdims=True) - xh * (gw * xh).sum(axis=-1, keepdims=True))
    return dx.astype(f32), (g64 * xh).reshape(-1, d).sum(0).astype(f32), g64.reshape(-1, d).sum(0).astype(f32)


# ---------------------------------------------------------------- activations
_K0, _K1 = 0.7978845608, 0.044715


def gelu_fwd(x):
    """ops::gelu core/ops.cpp:1243-1267 (tanh approximation)."""
    x = x.astype(np.float64)
    return (0.5 * x * (1.0 + np.tanh(_K0 * (x + _K1 * x ** 3)))).astype(f32)


def gelu_grad(x):
    """GeluBackward core/backward_functions.cpp:164-186."""
    x = x.astype(np.float64)
    t = np.tanh(_K0 * (x + _K1 * x ** 3))
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * _K0 * (1.0 + 3.0 * _K1 * x * x)


def swiglu_fwd(gate, up):
    """ops::swiglu core/ops.cpp:2416-2452."""
    g = gate.astype(np.float64)
    return (g / (1.0 + np.exp(-g)) * up).astype(f32)


def swiglu_bwd(dy, gate, up):
    """SwiGLUBackward core/backward_functions.cpp:277-295."""
    g, u, d = gate.astype(np.float64), up.astype(np.float64), dy.astype(np.float64)
    s = 1.0 / (1.0 + np.exp(-g))
    return (d * u * s * (1.0 + g * (1.0 - s))).astype(f32), (d * g * s).astype(f32)


def geglu_fwd(gate, up):
    """Gemma MLP: mul(gelu(gate), up), graph/gemma_model.cpp:538-546."""
    return (gelu_fwd(gate).astype(np.float64) * up).astype(f32)


def geglu_bwd(dy, gate, up):
    d = dy.astype(np.float64)
    return (d * up * gelu_grad(gate)).astype(f32), (d * gelu_fwd(gate)).astype(f32)


# ---------------------------------------------------------------- loss
def lm_cross_entropy(logits, labels, ignore_index=-100):
    """lm_cross_entropy core/lm_loss.cpp:268-382 and LMCrossEntropyBackward :75-163 ("mean").
    Row (b, s < S-1) is scored against labels[b, s+1].  Returns (loss, dlogits, n_valid)."""
    b, s, v = logits.shape
    z = logits[:, :-1, :].astype(np.float64)
    y = labels[:, 1:]
    valid = y != ignore_index
    if np.any(valid & ((y < 0) | (y >= v))):
        raise IndexError("lm_cross_entropy: label out of range")
    m = z.max(axis=-1, keepdims=True)
    e = np.exp(z - m)
    denom = e.sum(axis=-1, keepdims=True)
    lse = (m + np.log(denom))[..., 0]
    ysafe = np.where(valid, y, 0)
    picked = np.take_along_axis(z, ysafe[..., None], axis=-1)[..., 0]
    n = int(valid.sum())
    loss = f32(((lse - picked) * valid).sum() / n) if n > 0 else f32(np.nan)
    p = e / denom
    onehot = np.zeros_like(p)
    np.put_along_axis(onehot, ysafe[..., None], 1.0, axis=-1)
    coeff = (1.0 / n) if n > 0 else 0.0
    g = (p - onehot) * valid[..., None] * coeff
    dlogits = np.zeros((b, s, v), dtype=f32)
    dlogits[:, :-1, :] = g.astype(f32)
    return loss, dlogits, n


def lm_head_ce(hidden, table, labels, ignore_index=-100):
    """matmul_rhs_T(hidden, table) then lm_cross_entropy; returns (loss, dhidden)."""
    logits = (hidden.astype(np.float64) @ table.astype(np.float64).T).astype(f32)
    loss, dlogits, _ = lm_cross_entropy(logits, labels, ignore_index)
    dh = (dlogits.astype(np.float64) @ table.astype(np.float64)).astype(f32)
    return loss, dh


# ---------------------------------------------------------------- optimizer
def clip_scale(grads, max_norm, clip_eps=0.0):
    """Optimizer::clip_grad_norm optim/optimizer.cpp:6-38 (clip_eps=0) or the trainers' variant (1e-6)."""
    total = f32(0)
    for g in grads:
        total += (g.astype(f32) ** 2).sum(dtype=f32)
    norm = np.sqrt(total)
    if max_norm > 0 and norm > max_norm:
        return f32(max_norm) / (norm + f32(clip_eps))
    return f32(1.0)


def adam_step(p, g, m, v, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
    """Adam::step optim/adam.cpp:25-90: L2-style decay, bias correction 1 - powf(beta, step), eps outside sqrt."""
    p, g, m, v = (a.astype(f32) for a in (p, g, m, v))
    lr, beta1, beta2, eps = f32(lr), f32(beta1), f32(beta2), f32(eps)
    if weight_decay > 0:
        g = g + f32(weight_decay) * p
    m = beta1 * m + (f32(1) - beta1) * g
    v = beta2 * v + (f32(1) - beta2) * g * g
    bc1 = f32(1) - np.power(beta1, f32(step), dtype=f32)
    bc2 = f32(1) - np.power(beta2, f32(step), dtype=f32)
    p = p - lr * (m / bc1) / (np.sqrt(v / bc2) + eps)
    return p.astype(f32), m.astype(f32), v.astype(f32)


def embedding(ids, table, scale=1.0, pos_table=None):
    """Row gather (graph/gemma_model.cpp:222-259 with scale sqrtf(hidden); gpt2 adds positions :349-369)."""
    if np.any((ids < 0) | (ids >= table.shape[0])):
        raise IndexError("embedding_lookup: token id out of range")
    out = table[ids] * f32(scale)
    if pos_table is not None:
        out = out + pos_table[np.arange(ids.shape[1])][None, :, :]
    return out.astype(f32)


def trainer_lr(step, learning_rate, warmup_ratio, lr_scheduler, total_updates):
    """get_lr of the trainers (optim/gemma_trainer.cpp:44-62, optim/trainer.cpp:46-73) for optimizer step `step`
    (1-based), with float32 arithmetic where the reference uses float.  `lr_scheduler`: "linear", "cosine" or any
    other name (GemmaLoRATrainer: linear; LoRATrainer: constant after the warm-up -> pass "constant")."""
    f = np.float32
    total = max(1, int(total_updates))
    warmup_steps = int(f(total) * f(warmup_ratio))          # int64 * float -> float, truncated
    if warmup_steps > 0 and step <= warmup_steps:
        return float(f(learning_rate) * (f(step) / f(warmup_steps)))
    progress = f(step - warmup_steps) / f(max(1, total - warmup_steps))
    progress = min(max(progress, f(0)), f(1))
    if lr_scheduler == "cosine":
        return float(f(learning_rate) * f(0.5) * (f(1) + f(np.cos(f(3.14159265) * progress))))
    if lr_scheduler == "linear":
        return float(f(learning_rate) * (f(1) - progress))
    return float(f(learning_rate))


def ppl_accumulate(batch_losses, batch_labels):
    """Aggregation of examples/gpt2_small_lora_finetune/src/eval_ppl.cpp:166-210: each batch's float mean loss is
    weighted by the count of labels != -100 in the whole (unshifted) labels tensor, float * int64 -> float, summed
    in double; returns (mean_nll float32, ppl = exp(mean_nll) float32, tokens)."""
    sum_loss, sum_tokens = 0.0, 0
    for loss, labels in zip(batch_losses, batch_labels):
        valid = int((np.asarray(labels) != -100).sum())
        sum_loss += float(np.float32(loss) * np.float32(valid))
        sum_tokens += valid
    mean_nll = np.float32(sum_loss / sum_tokens) if sum_tokens > 0 else np.float32(0)
    return float(mean_nll), float(np.exp(mean_nll, dtype=np.float32)), sum_tokens
