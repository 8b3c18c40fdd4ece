"""Operator-level wrappers over the C ABI, taking torch CUDA tensors.

torch only provides device memory and the current stream here; every
computation happens in libmft_cuda.so.  The wrappers mirror the reference's
`ops::` functions on the LoRA step's path (operator/finetune_ops/core/ops.h,
lm_loss.h, optim/adam.h) so that the parity tests read like the reference's.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib as L

BF16, F32 = torch.bfloat16, torch.float32


def _dt(t: torch.Tensor) -> int:
    if t.dtype == F32:
        return L.MFT_F32
    if t.dtype == BF16:
        return L.MFT_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _init(t: torch.Tensor):
    if not t.is_cuda:
        raise L.MftError("mobilefinetuner_b200 has no CPU path: tensors must live on a CUDA device")
    L.init(t.device.index or 0)


def device_status() -> int:
    s = C.c_int32(0)
    L.call("mft_device_status", _stream(), C.byref(s))
    return s.value


# ---------------------------------------------------------------- GEMMs
def gemm_nt(a, b, *, a2=None, b2=None, bias=None, alpha=1.0, out=None, out_dtype=BF16, accumulate=False):
    """D = alpha * (A @ B^T + A2 @ B2^T) + bias (+ D).  A [M,K], B [N,K] bf16."""
    _init(a)
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty(m, n, device=a.device, dtype=out_dtype)
    k2 = 0 if a2 is None else a2.shape[1]
    L.call("mft_gemm_nt", _p(a), a.stride(0), _p(b), b.stride(0), m, n, k,
           _p(a2), 0 if a2 is None else a2.stride(0), _p(b2), 0 if b2 is None else b2.stride(0), k2,
           _p(bias), float(alpha), _p(out), out.stride(0), _dt(out), 1 if accumulate else 0, _stream())
    return out


def gemm_nt_tile_cols(m, n, k, k2=0, out_dtype=BF16):
    """Columns of the CTA-pair kernel's tile for a gemm_nt call of this shape (256 / 384), 0 when another kernel runs it."""
    L.init(torch.cuda.current_device())
    cols = C.c_int32(0)
    L.call("mft_gemm_nt_tile_cols", m, n, k, k2, L.MFT_BF16 if out_dtype == BF16 else L.MFT_F32, C.byref(cols))
    return cols.value


def gemm_tn_acc(u, v, out, alpha=1.0):
    """out[P,Q] += alpha * U^T V with U [T,P], V [T,Q] bf16, out f32."""
    _init(u)
    t, p = u.shape
    q = v.shape[1]
    L.call("mft_gemm_tn_acc", _p(u), u.stride(0), _p(v), v.stride(0), t, p, q, float(alpha), _p(out), out.stride(0), _stream())
    return out


# ---------------------------------------------------------------- norms
def rms_norm_fwd(x, weight, eps, unit_offset, out_dtype=BF16, residual=None):
    _init(x)
    rows, dim = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty(x.shape, device=x.device, dtype=out_dtype)
    rstd = torch.empty(rows, device=x.device, dtype=F32)
    sum_out = torch.empty(x.shape, device=x.device, dtype=F32) if residual is not None else None
    L.call("mft_rmsnorm_fwd", _p(x), _dt(x), _p(weight), float(eps), int(unit_offset), _p(y), _dt(y), _p(rstd),
           _p(residual), _p(sum_out), rows, dim, _stream())
    return (y, rstd, sum_out) if residual is not None else (y, rstd)


def rms_norm_bwd(dy, x, weight, rstd, eps, unit_offset, out_dtype=F32, dweight=None, accumulate_into=None):
    _init(x)
    rows, dim = x.numel() // x.shape[-1], x.shape[-1]
    dx = accumulate_into if accumulate_into is not None else torch.empty(x.shape, device=x.device, dtype=out_dtype)
    L.call("mft_rmsnorm_bwd", _p(dy), _dt(dy), _p(x), _dt(x), _p(weight), _p(rstd), float(eps), int(unit_offset),
           _p(dx), _dt(dx), 1 if accumulate_into is not None else 0, _p(dweight), rows, dim, _stream())
    return dx


def rms_norm_add_norm_fwd(y, w_post, residual, w_next, eps, unit_post=1, unit_next=1):
    """sum = residual + rms_norm(y; w_post), h = rms_norm(sum; w_next) in one pass: returns (sum, rstd_post, h, rstd_next)."""
    _init(y)
    rows, dim = y.numel() // y.shape[-1], y.shape[-1]
    sum_out = torch.empty(y.shape, device=y.device, dtype=F32)
    h = torch.empty(y.shape, device=y.device, dtype=BF16)
    rp = torch.empty(rows, device=y.device, dtype=F32)
    rn = torch.empty(rows, device=y.device, dtype=F32)
    L.call("mft_rmsnorm_add_norm_fwd", _p(y), _p(w_post), int(unit_post), _p(residual), _p(w_next), int(unit_next), float(eps),
           _p(sum_out), _p(rp), _p(h), _p(rn), rows, dim, _stream())
    return sum_out, rp, h, rn


def rms_norm_pair_bwd(dy_next, x_sum, w_next, rstd_next, dx_inout, y_branch, w_post, rstd_post, unit_post=1, unit_next=1):
    """dx_inout += d rms_norm(x_sum; w_next)(dy_next); returns d rms_norm(y_branch; w_post)(dx_inout) as bf16."""
    _init(x_sum)
    rows, dim = x_sum.numel() // x_sum.shape[-1], x_sum.shape[-1]
    d_branch = torch.empty(y_branch.shape, device=x_sum.device, dtype=BF16)
    L.call("mft_rmsnorm_pair_bwd", _p(dy_next), _p(x_sum), _p(w_next), int(unit_next), _p(rstd_next), _p(dx_inout), _p(y_branch),
           _p(w_post), int(unit_post), _p(rstd_post), _p(d_branch), rows, dim, _stream())
    return d_branch


def layer_norm_fwd(x, weight, bias, eps, out_dtype=BF16):
    _init(x)
    rows, dim = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty(x.shape, device=x.device, dtype=out_dtype)
    mean = torch.empty(rows, device=x.device, dtype=F32)
    rstd = torch.empty(rows, device=x.device, dtype=F32)
    L.call("mft_layernorm_fwd", _p(x), _dt(x), _p(weight), _p(bias), float(eps), _p(y), _dt(y), _p(mean), _p(rstd), rows, dim, _stream())
    return y, mean, rstd


def layer_norm_bwd(dy, x, weight, mean, rstd, out_dtype=F32, dweight=None, dbias=None):
    _init(x)
    rows, dim = x.numel() // x.shape[-1], x.shape[-1]
    dx = torch.empty(x.shape, device=x.device, dtype=out_dtype)
    L.call("mft_layernorm_bwd", _p(dy), _dt(dy), _p(x), _dt(x), _p(weight), _p(mean), _p(rstd), _p(dx), _dt(dx), 0,
           _p(dweight), _p(dbias), rows, dim, _stream())
    return dx


# ---------------------------------------------------------------- activations
def act_fwd(kind, gate, up=None):
    _init(gate)
    rows, cols = gate.shape
    y = torch.empty(rows, cols, device=gate.device, dtype=BF16)
    L.call("mft_act_fwd", kind, _p(gate), _p(up), gate.stride(0), _p(y), rows, cols, _stream())
    return y


def act_bwd(kind, dy, gate, up=None):
    _init(gate)
    rows, cols = gate.shape
    dgate = torch.empty_strided(gate.shape, gate.stride(), device=gate.device, dtype=BF16)
    dup = torch.empty_strided(gate.shape, gate.stride(), device=gate.device, dtype=BF16) if up is not None else None
    L.call("mft_act_bwd", kind, _p(dy), _p(gate), _p(up), gate.stride(0), _p(dgate), _p(dup), rows, cols, _stream())
    return dgate, dup


def glu_linear_fwd(kind, x, w_nk, *, xa=None, b_nk=None, bias=None):
    """Gated MLP, forward, gating fused into the GEMM epilogue: returns (gate|up [M, 2I], act [M, I]) or None when the
    shape does not qualify for the fused kernel.  w_nk [2I, K] (gate rows first), xa [M, r], b_nk [2I, r]."""
    _init(x)
    m, k = x.shape
    inter = w_nk.shape[0] // 2
    gu = torch.empty(m, 2 * inter, device=x.device, dtype=BF16)
    act = torch.empty(m, inter, device=x.device, dtype=BF16)
    k2 = 0 if xa is None else xa.shape[1]
    rc = L.load().mft_glu_linear_fwd(kind, _p(x), x.stride(0), _p(w_nk), w_nk.stride(0), m, inter, k, _p(xa), 0 if xa is None else xa.stride(0),
                                     _p(b_nk), 0 if b_nk is None else b_nk.stride(0), k2, _p(bias), _p(gu), gu.stride(0), _p(act), act.stride(0), _stream())
    if rc == L.MFT_ERR_UNSUPPORTED:
        return None
    if rc != 0:
        raise L.MftError(f"mft_glu_linear_fwd failed with status {rc}: {L.load().mft_last_error().decode(errors='replace')}")
    return gu, act


def glu_linear_bwd(kind, dy, w_kn, gu, *, a2=None, b2=None):
    """Gated MLP, backward through the down projection and the gating in one launch: d_gate|d_up [M, 2I] from dy [M, K],
    the down-projection weight w_kn [I, K] (K-major) and the saved gate|up; None when the shape does not qualify."""
    _init(dy)
    m, k = dy.shape
    inter = w_kn.shape[0]
    dgu = torch.empty(m, 2 * inter, device=dy.device, dtype=BF16)
    k2 = 0 if a2 is None else a2.shape[1]
    rc = L.load().mft_glu_linear_bwd(kind, _p(dy), dy.stride(0), _p(w_kn), w_kn.stride(0), m, inter, k, _p(a2), 0 if a2 is None else a2.stride(0),
                                     _p(b2), 0 if b2 is None else b2.stride(0), k2, _p(gu), gu.stride(0), _p(dgu), dgu.stride(0), _stream())
    if rc == L.MFT_ERR_UNSUPPORTED:
        return None
    if rc != 0:
        raise L.MftError(f"mft_glu_linear_bwd failed with status {rc}: {L.load().mft_last_error().decode(errors='replace')}")
    return dgu


# ---------------------------------------------------------------- RoPE (+ per-head norm)
def rope_tables(seq_len, head_dim, theta, device):
    cos = torch.empty(seq_len, head_dim // 2, dtype=F32)
    sin = torch.empty(seq_len, head_dim // 2, dtype=F32)
    L.call("mft_rope_table_host", cos.data_ptr(), sin.data_ptr(), seq_len, head_dim, float(theta))
    return cos.to(device), sin.to(device)


def headnorm_rope_fwd(x, seq_len, n_heads, head_dim, cos=None, sin=None, norm_weight=None, eps=1e-6):
    """x: bf16 [tokens, n_heads*head_dim] (row stride may exceed the width)."""
    _init(x)
    tokens = x.shape[0]
    y = torch.empty(tokens, n_heads * head_dim, device=x.device, dtype=BF16)
    rstd = torch.empty(tokens * n_heads, device=x.device, dtype=F32) if norm_weight is not None else None
    L.call("mft_headnorm_rope_fwd", _p(x), x.stride(0), _p(norm_weight), float(eps), _p(cos), _p(sin), _p(y), y.stride(0),
           _p(rstd), tokens, seq_len, n_heads, head_dim, _stream())
    return y, rstd


def headnorm_rope_bwd(dy, x, seq_len, n_heads, head_dim, cos=None, sin=None, norm_weight=None, rstd=None):
    _init(dy)
    tokens = dy.shape[0]
    dx = torch.empty(tokens, n_heads * head_dim, device=dy.device, dtype=BF16)
    L.call("mft_headnorm_rope_bwd", _p(dy), dy.stride(0), _p(x), 0 if x is None else x.stride(0), _p(norm_weight), _p(rstd),
           _p(cos), _p(sin), _p(dx), dx.stride(0), tokens, seq_len, n_heads, head_dim, _stream())
    return dx


# ---------------------------------------------------------------- attention
def _strides_bhsd(t):
    """t: [B, H, S, D] view (any strides with unit stride on D)."""
    assert t.stride(3) == 1
    return L.Strides(t.stride(0), t.stride(2), t.stride(1))


def attention_fwd(q, k, v, scale, window=0):
    """q [B,nh,S,hd], k/v [B,nkv,S,hd] bf16 views (last dim contiguous) -> O like q, lse [B,nh,S]."""
    _init(q)
    b, nh, s, hd = q.shape
    nkv = k.shape[1]
    o = torch.empty_strided(q.shape, q.stride(), device=q.device, dtype=BF16)
    lse = torch.empty(b, nh, s, device=q.device, dtype=F32)
    L.call("mft_attn_fwd", _p(q), _strides_bhsd(q), _p(k), _strides_bhsd(k), _p(v), _strides_bhsd(v), _p(o), _strides_bhsd(o),
           _p(lse), b, s, nh, nkv, hd, float(scale), int(window), _stream())
    return o, lse


def attention_bwd(q, k, v, o, d_o, lse, scale, window=0, split_heads=True):
    """dQ, dK, dV.  With grouped KV heads and split_heads, each query head runs in its own CTAs and adds its
    dK/dV share into an f32 scratch; otherwise one CTA walks the whole group."""
    _init(q)
    b, nh, s, hd = q.shape
    nkv = k.shape[1]
    acc = torch.empty(2 * b * s * nkv * hd, device=q.device, dtype=F32) if (split_heads and nh > nkv) else None
    dq = torch.empty_strided(q.shape, q.stride(), device=q.device, dtype=BF16)
    dk = torch.empty_strided(k.shape, k.stride(), device=q.device, dtype=BF16)
    dv = torch.empty_strided(v.shape, v.stride(), device=q.device, dtype=BF16)
    delta = torch.empty(b, nh, s, device=q.device, dtype=F32)
    L.call("mft_attn_bwd", _p(q), _strides_bhsd(q), _p(k), _strides_bhsd(k), _p(v), _strides_bhsd(v), _p(o), _strides_bhsd(o),
           _p(d_o), _strides_bhsd(d_o), _p(lse), _p(dq), _p(dk), _p(dv), _p(delta), _p(acc) if acc is not None else None,
           b, s, nh, nkv, hd, float(scale), int(window), _stream())
    return dq, dk, dv


def attention_bwd_noalloc(q, k, v, o, d_o, lse, scale, window=0):
    """attention_bwd for callers that cannot allocate device memory: the row-sum scratch is a fixed
    array inside the library (at most 2**20 rows = batch * heads * seq).  The outputs are written
    into tensors the caller made beforehand; here they are created up front only for convenience."""
    _init(q)
    b, nh, s, hd = q.shape
    nkv = k.shape[1]
    dq = torch.empty_strided(q.shape, q.stride(), device=q.device, dtype=BF16)
    dk = torch.empty_strided(k.shape, k.stride(), device=q.device, dtype=BF16)
    dv = torch.empty_strided(v.shape, v.stride(), device=q.device, dtype=BF16)
    L.call("mft_attn_bwd_noalloc", _p(q), _strides_bhsd(q), _p(k), _strides_bhsd(k), _p(v), _strides_bhsd(v), _p(o), _strides_bhsd(o),
           _p(d_o), _strides_bhsd(d_o), _p(lse), _p(dq), _p(dk), _p(dv), b, s, nh, nkv, hd, float(scale), int(window), _stream())
    return dq, dk, dv


# ---------------------------------------------------------------- lm head + CE
class LmHeadCE:
    """Shifted-label cross entropy over hidden x table^T (the logits never hit memory)."""

    def __init__(self, table_bf16: torch.Tensor):
        _init(table_bf16)
        self.table = table_bf16.contiguous()
        v, h = self.table.shape
        self.ld_t = (v + 63) // 64 * 64
        self.table_t = torch.zeros(h, self.ld_t, device=table_bf16.device, dtype=BF16)
        tmp = torch.empty(h, v, device=table_bf16.device, dtype=BF16)
        L.call("mft_transpose_bf16", _p(self.table), _p(tmp), v, h, _stream())
        self.table_t[:, :v] = tmp
        self._ws = None

    def _workspace(self, t, h, v):
        need = L.call("mft_lmhead_ce_workspace_bytes", t, h, v)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, device=self.table.device, dtype=torch.uint8)
        return self._ws

    def forward(self, hidden, labels, ignore_index=-100):
        b, s, h = hidden.shape
        v = self.table.shape[0]
        ws = self._workspace(b * s, h, v)
        dev = hidden.device
        self.loss = torch.empty(1, device=dev, dtype=F32)
        self.n_valid = torch.zeros(1, device=dev, dtype=torch.int32)
        self.lse = torch.empty(b * s, device=dev, dtype=F32)
        self.status = torch.zeros(1, device=dev, dtype=torch.int32)
        L.call("mft_lmhead_ce_fwd", _p(hidden), _p(self.table), _p(labels), b, s, h, v, ignore_index, _p(self.loss),
               _p(self.n_valid), _p(self.lse), _p(self.status), _p(ws), ws.numel(), _stream())
        if int(self.status.item()) != 0:
            raise IndexError("lm_cross_entropy: label out of range")
        return self.loss

    def backward(self, hidden, labels, dloss=1.0, ignore_index=-100, n_valid_override=0):
        b, s, h = hidden.shape
        v = self.table.shape[0]
        ws = self._workspace(b * s, h, v)
        dh = torch.empty(b, s, h, device=hidden.device, dtype=BF16)
        L.call("mft_lmhead_ce_bwd", _p(hidden), _p(self.table), _p(self.table_t), self.ld_t, _p(labels), b, s, h, v,
               ignore_index, _p(self.lse), _p(self.n_valid), int(n_valid_override), float(dloss), _p(dh), _p(ws), ws.numel(), _stream())
        return dh


    def fused(self, hidden, labels, dloss=1.0, ignore_index=-100, n_valid_override=0):
        """Loss and d(loss)/d(hidden) from one sweep over the vocabulary: returns (loss, dhidden)."""
        b, s, h = hidden.shape
        v = self.table.shape[0]
        ws = self._workspace(b * s, h, v)
        dev = hidden.device
        self.loss = torch.empty(1, device=dev, dtype=F32)
        self.n_valid = torch.zeros(1, device=dev, dtype=torch.int32)
        self.lse = torch.empty(b * s, device=dev, dtype=F32)
        self.status = torch.zeros(1, device=dev, dtype=torch.int32)
        dh = torch.empty(b, s, h, device=dev, dtype=BF16)
        L.call("mft_lmhead_ce_fused", _p(hidden), _p(self.table), _p(self.table_t), self.ld_t, _p(labels), b, s, h, v,
               ignore_index, int(n_valid_override), float(dloss), _p(self.loss), _p(self.n_valid), _p(self.lse), _p(dh),
               _p(self.status), _p(ws), ws.numel(), _stream())
        if int(self.status.item()) != 0:
            raise IndexError("lm_cross_entropy: label out of range")
        return self.loss, dh


def ce_dense(logits, labels, ignore_index=-100, dloss=1.0):
    """lm_cross_entropy on dense f32 logits [B,S,V]: returns (loss, dlogits)."""
    _init(logits)
    b, s, v = logits.shape
    dev = logits.device
    loss = torch.empty(1, device=dev, dtype=F32)
    n_valid = torch.zeros(1, device=dev, dtype=torch.int32)
    lse = torch.empty(b * s, device=dev, dtype=F32)
    tgt = torch.empty(b * s, device=dev, dtype=torch.int32)
    acc = torch.zeros(1, device=dev, dtype=torch.float64)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    L.call("mft_ce_dense_fwd", _p(logits), _p(labels), b, s, v, ignore_index, _p(loss), _p(n_valid), _p(lse), _p(tgt), _p(acc), _p(status), _stream())
    if int(status.item()) != 0:
        raise IndexError("lm_cross_entropy: label out of range")
    dlogits = torch.empty_like(logits)
    L.call("mft_ce_dense_bwd", _p(logits), _p(tgt), b, s, v, _p(lse), _p(n_valid), float(dloss), _p(dlogits), _stream())
    return loss, dlogits


# ---------------------------------------------------------------- misc
def embedding_gather(ids, table_bf16, scale=1.0, pos_table=None, seq_len=None):
    _init(table_bf16)
    n = ids.numel()
    v, h = table_bf16.shape
    out = torch.empty(n, h, device=table_bf16.device, dtype=F32)
    status = torch.zeros(1, device=table_bf16.device, dtype=torch.int32)
    L.call("mft_embedding_gather", _p(ids), _p(table_bf16), _p(pos_table), _p(out), n, seq_len or n, h, v, float(scale), _p(status), _stream())
    if int(status.item()) != 0:
        raise IndexError("embedding_lookup: token id out of range")
    return out


def repeat_kv(kv, repeat):
    _init(kv)
    b, nkv, s, hd = kv.shape
    out = torch.empty(b, nkv * repeat, s, hd, device=kv.device, dtype=kv.dtype)
    L.call("mft_repeat_kv", _p(kv), _dt(kv), _p(out), b, nkv, s, hd, repeat, _stream())
    return out


def repeat_kv_bwd(dout, repeat):
    _init(dout)
    b, nh, s, hd = dout.shape
    dkv = torch.empty(b, nh // repeat, s, hd, device=dout.device, dtype=F32)
    L.call("mft_repeat_kv_bwd", _p(dout), _p(dkv), b, nh // repeat, s, hd, repeat, _stream())
    return dkv


def adam_step(params, grads, m, v, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
              max_norm=0.0, clip_eps=0.0, zero_grad=True):
    _init(params)
    n = params.numel()
    sq = torch.zeros(1, device=params.device, dtype=F32)
    L.call("mft_grad_sqnorm", _p(grads), n, _p(sq), _stream())
    L.call("mft_adam_step", _p(params), _p(grads), _p(m), _p(v), n, int(step), float(lr), float(beta1), float(beta2),
           float(eps), float(weight_decay), _p(sq), float(max_norm), float(clip_eps), 1 if zero_grad else 0, _stream())
    return sq
