"""Seeded random-shape sweep of the CUDA operators (GEMM with the LoRA k-block / bias / f32 accumulate, the
token-contracting GEMM on both of its kernels, attention on the mma.sync and the tcgen05 kernels, the lm-head
cross entropy in one and two sweeps) against float64 references evaluated with torch on the same device.  The fixed
shapes of the other test files pin values against the oracle; this file covers the ragged shapes in between:
odd row counts, widths that end inside a tile, windows of every length, vocabularies that are no multiple of 8."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16
dev = "cuda"


@pytest.fixture(scope="module")
def ops():
    from mobilefinetuner_b200 import ops as O
    return O


class Sweep:
    def __init__(self, ops, seed):
        self.ops = ops
        self.g = np.random.Generator(np.random.PCG64(seed))
        self.tg = torch.Generator(device=dev); self.tg.manual_seed(seed)
        self.fails = []

    def rnd(self, *shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=self.tg) * scale).to(BF)

    def check(self, name, cfg, err, lim):
        if not (err < lim):
            self.fails.append((name, cfg, err))


def relerr(a, b, floor=0.0):
    a, b = a.double(), b.double()
    return float((a - b).norm() / max(float(b.norm()) + floor * b.numel() ** 0.5, 1e-30))


def sweep_gemm(sw):
    g, tg, ops, rnd, check = sw.g, sw.tg, sw.ops, sw.rnd, sw.check
    m = int(g.integers(1, 900)); n = int(g.integers(1, 200)) * 8; k = int(g.integers(1, 400)) * 8
    use2 = bool(g.integers(0, 2)); k2 = int(g.choice([16, 32, 48, 64]))
    bias = bool(g.integers(0, 2)); f32 = bool(g.integers(0, 2)); alpha = float(g.choice([1.0, 0.5, 2.0]))
    a, b = rnd(m, k), rnd(n, k, scale=0.05)
    a2 = rnd(m, 64) if use2 else None; b2 = rnd(n, 64, scale=0.05) if use2 else None
    if use2:
        a2[:, k2:] = 0; b2[:, k2:] = 0
        a2v, b2v = a2[:, :k2], b2[:, :k2]
    bs = torch.randn(n, device=dev, generator=tg) if bias else None
    want = a.double() @ b.double().T
    if use2:
        want = want + a2.double() @ b2.double().T
    want = alpha * want
    if bias:
        want = want + bs.double()
    out = ops.gemm_nt(a, b, a2=a2v if use2 else None, b2=b2v if use2 else None, bias=bs, alpha=alpha, out_dtype=torch.float32 if f32 else BF)
    check("gemm_nt", (m, n, k, use2, k2, bias, f32, alpha), relerr(out, want), 1e-5 if f32 else 4e-3)
    if f32 and not bias:
        base = torch.randn(m, n, device=dev, generator=tg)
        out2 = base.clone()
        ops.gemm_nt(a, b, alpha=alpha, out=out2, accumulate=True)
        check("gemm_nt_acc", (m, n, k), relerr(out2, base.double() + alpha * (a.double() @ b.double().T)), 1e-5)


def sweep_tn(sw):
    g, tg, ops, rnd, check = sw.g, sw.tg, sw.ops, sw.rnd, sw.check
    # P >= 2048 takes the tcgen05 kernel, narrower ones the mma.sync kernel
    t = int(g.integers(1, 6000)); p = int(g.integers(8, 400)) * 8; q = int(g.choice([8, 16, 24, 48, 64, 128, 200]))
    wide = int(g.choice([64, 128, 256])) if q <= 64 else q
    u = rnd(t, p); vbuf = rnd(t, max(wide, q)); v = vbuf[:, :q]
    swap = bool(g.integers(0, 2))
    if swap:
        out = torch.zeros(q, p, device=dev); ops.gemm_tn_acc(v, u, out, alpha=0.5)
        want = 0.5 * (v.double().T @ u.double())
    else:
        out = torch.zeros(p, q, device=dev); ops.gemm_tn_acc(u, v, out, alpha=0.5)
        want = 0.5 * (u.double().T @ v.double())
    check("gemm_tn", (t, p, q, wide, swap), relerr(out, want), 2e-5)


def attn_ref(q, k, v, dO, scale, window):
    B, nh, S, hd = q.shape
    nkv = k.shape[1]; rep = nh // nkv
    qd, kd, vd, dOd = (x.double() for x in (q, k, v, dO))
    kk = kd.repeat_interleave(rep, 1); vv = vd.repeat_interleave(rep, 1)
    s = (qd @ kk.transpose(-1, -2)) * scale
    i = torch.arange(S, device=dev)[:, None]; j = torch.arange(S, device=dev)[None, :]
    mask = j <= i
    if window > 0:
        mask = mask & (i - j < window)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    o = p @ vv
    dv = p.transpose(-1, -2) @ dOd
    dp = dOd @ vv.transpose(-1, -2)
    delta = (o * dOd).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kk
    dk = ds.transpose(-1, -2) @ qd
    dk = dk.view(B, nkv, rep, S, hd).sum(2); dv = dv.view(B, nkv, rep, S, hd).sum(2)
    return o, dq, dk, dv


def sweep_attn(sw):
    g, tg, ops, rnd, check = sw.g, sw.tg, sw.ops, sw.rnd, sw.check
    hd = int(g.choice([256, 256, 64, 128]))
    B = int(g.integers(1, 4)); nkv = int(g.choice([1, 2])); rep = int(g.choice([1, 2, 4])); nh = nkv * rep
    if hd == 256 and g.integers(0, 4) > 0:
        S = int(g.integers(1, 9)) * 128          # the tcgen05 kernels
    else:
        S = int(g.integers(24, 700))             # the mma.sync kernels (any length)
    window = 0 if g.integers(0, 2) else int(g.integers(1, S + 1))
    amp = float(g.choice([1.0, 1.0, 3.0]))

    def tok(*shape):   # token-major storage viewed [B,H,S,D]
        Bq, H, Sq, D = shape
        return (torch.randn(Bq, Sq, H, D, device=dev, generator=tg)).to(BF).permute(0, 2, 1, 3)
    q, k, v, dO = tok(B, nh, S, hd), tok(B, nkv, S, hd), tok(B, nkv, S, hd), tok(B, nh, S, hd)
    if amp > 1:
        q = (q.float() * amp).to(BF); k = (k.float() * amp).to(BF)
    scale = hd ** -0.5
    o, lse = ops.attention_fwd(q, k, v, scale, window)
    dq, dk, dv = ops.attention_bwd(q, k, v, o, dO, lse, scale, window)
    wo, wdq, wdk, wdv = attn_ref(q, k, v, dO, scale, window)
    cfg = (hd, B, nkv, rep, S, window, amp)
    for nm, a, b in (("o", o, wo), ("dq", dq, wdq), ("dk", dk, wdk), ("dv", dv, wdv)):
        # absolute floor of 4e-3 * amp per element: where a query sees one key (window 1) or its softmax is one-hot,
        # dS is 0 in exact arithmetic and what is left is the bf16 rounding of the stored O in rowsum(O dO)
        check("attn_" + nm, cfg, relerr(a, b, floor=4e-3 * amp), 2e-2)
    check("attn_status", cfg, ops.device_status(), 1)


def sweep_ce(sw):
    g, tg, ops, rnd, check = sw.g, sw.tg, sw.ops, sw.rnd, sw.check
    t = int(g.integers(1, 700)); h = int(g.choice([64, 128, 256, 640, 896])); v = int(g.integers(100, 50000))
    B = 1
    W = rnd(v, h, scale=float(g.choice([0.02, 0.2])))
    hid = rnd(B, t, h, scale=float(g.choice([1.0, 3.0])))
    labels = torch.randint(0, v, (B, t), device=dev, dtype=torch.int32, generator=tg)
    nign = int(g.integers(0, max(1, t // 3)))
    if nign:
        labels[0, :nign] = -100
    ce = ops.LmHeadCE(W)
    loss, dh = ce.fused(hid, labels, dloss=1.0)
    logits = hid.double().view(t, h) @ W.double().T
    lab = labels.view(-1).long()
    # shifted labels: position i predicts labels[i+1]
    tgt = torch.full((t,), -100, device=dev, dtype=torch.long)
    tgt[:-1] = lab[1:]
    valid = tgt != -100
    nv = int(valid.sum())
    if nv == 0:
        return
    lsm = torch.log_softmax(logits, -1)
    want_loss = -(lsm[valid, tgt[valid]]).sum() / nv
    p = torch.softmax(logits, -1)
    gl = p.clone()
    gl[valid, tgt[valid]] -= 1
    gl[~valid] = 0
    gl = gl / nv
    want_dh = gl @ W.double()
    cfg = (t, h, v, nign)
    check("ce_loss", cfg, abs(float(loss) - float(want_loss)) / max(abs(float(want_loss)), 1e-9), 2e-3)
    check("ce_dh", cfg, relerr(dh.view(t, h), want_dh), 2e-2)
    loss2 = ce.forward(hid, labels); dh2 = ce.backward(hid, labels)
    check("ce2_loss", cfg, abs(float(loss2) - float(want_loss)) / max(abs(float(want_loss)), 1e-9), 2e-3)
    check("ce2_dh", cfg, relerr(dh2.view(t, h), want_dh), 2e-2)




@pytest.mark.parametrize("kind,fn,cases", [("gemm", sweep_gemm, 1500), ("tn", sweep_tn, 1500), ("attn", sweep_attn, 1000), ("ce", sweep_ce, 400)])
def test_random_shapes(ops, kind, fn, cases):
    sw = Sweep(ops, {"gemm": 101, "tn": 202, "attn": 303, "ce": 404}[kind])
    for _ in range(cases):
        fn(sw)
    torch.cuda.synchronize()
    assert not sw.fails, f"{len(sw.fails)} of {cases} {kind} cases outside tolerance, first: {sw.fails[:5]}"
