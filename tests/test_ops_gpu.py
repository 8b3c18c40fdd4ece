"""GPU parity suite, operator level: every call goes through the C ABI of libmft_cuda.so
and is compared with (a) the committed outputs of the compiled reference
(tests/golden/ops_golden.npz) and (b) the pinned numpy restatement on other seeded
shapes.  Integer / indexing work must be bit-exact; bf16 tensor-core paths are held to
cosine >= 0.999 and max-norm relative error <= 2e-2 (the tolerance of the path's spec),
fp32 paths to 1e-5."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import restate as R

pytestmark = pytest.mark.gpu

BF16_REL, BF16_COS = 2e-2, 0.999


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.detach().float().cpu().numpy()


def rb(x):
    return R.bf16_round(np.asarray(x, np.float32))


def close_bf16(got, want, rel=BF16_REL, cos=BF16_COS):
    assert np.isfinite(got).all()
    assert cosine(got, want) >= cos, f"cosine {cosine(got, want)}"
    assert rel_err(got, want) <= rel, f"rel err {rel_err(got, want)}"


@pytest.fixture(scope="module")
def ops():
    from mobilefinetuner_b200 import ops as O
    return O


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (1, 8, 8), (130, 72, 200), (257, 1152, 640), (512, 1536, 1152),
                                   (384, 256, 6912), (100, 2304, 768)])
def test_gemm_nt_matches_float64(ops, m, n, k):
    g = np.random.Generator(np.random.PCG64(m * 7 + n * 3 + k))
    a, b = rb(g.standard_normal((m, k))), rb(g.standard_normal((n, k)))
    want = a.astype(np.float64) @ b.astype(np.float64).T
    got = host(ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16), out_dtype=torch.float32))
    assert rel_err(got, want) < 1e-5
    got16 = host(ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16)))
    close_bf16(got16, want, rel=6e-3)
    assert ops.device_status() == 0


def test_gemm_nt_lora_segment_bias_alpha_accumulate(ops):
    g = np.random.Generator(np.random.PCG64(5))
    m, n, k, r = 300, 200, 136, 16
    a, b = rb(g.standard_normal((m, k))), rb(g.standard_normal((n, k)))
    a2, b2 = rb(g.standard_normal((m, r))), rb(g.standard_normal((n, r)))
    bias = g.standard_normal(n).astype(np.float32)
    prev = g.standard_normal((m, n)).astype(np.float32)
    want = 0.5 * (a.astype(np.float64) @ b.T + a2.astype(np.float64) @ b2.T) + bias + prev
    # the second segment lives in 64-wide zero-padded panels, as the LoRA step stores it
    a2p = np.zeros((m, 64), np.float32); a2p[:, :r] = a2
    b2p = np.zeros((n, 64), np.float32); b2p[:, :r] = b2
    out = dev(prev)
    ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16), a2=dev(a2p, torch.bfloat16)[:, :r], b2=dev(b2p, torch.bfloat16)[:, :r],
                bias=dev(bias), alpha=0.5, out=out, accumulate=True)
    assert rel_err(host(out), want) < 1e-5


@pytest.mark.parametrize("m,n,k,accumulate", [(256, 192, 8192, False), (300, 200, 20000, True), (130, 1152, 4104, False), (512, 1152, 8192, False), (768, 384, 16384, True)])
def test_gemm_nt_f32_deep_k_is_split_and_reduced(ops, m, n, k, accumulate):
    """f32 outputs with a long K: ranges of K run as separate tiles whose partial sums are added in memory."""
    g = np.random.Generator(np.random.PCG64(k + m))
    a, b = rb(g.standard_normal((m, k))), rb(g.standard_normal((n, k)))
    bias = g.standard_normal(n).astype(np.float32)
    prev = g.standard_normal((m, n)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64).T + bias + (prev if accumulate else 0.0)
    out = dev(prev)
    ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16), bias=dev(bias), out=out, accumulate=accumulate)
    assert rel_err(host(out), want) < 1e-5
    assert ops.device_status() == 0


@pytest.mark.parametrize("m,n,k,r", [(4096, 1152, 4096, 16), (8192, 768, 4128, 32), (4096, 1152, 8192, 0), (16384, 384, 4096, 0),
                                     (16384, 640, 2048, 8), (16384, 1000, 4096, 8)])   # the last two: a ragged last column tile
def test_gemm_nt_wide_tile_long_k(ops, m, n, k, r):
    """Outputs whose width is a multiple of 384 under K >= 4096 run on 256 x 384 tiles with one accumulator buffer
    (two 192-column MMAs per k-step) when the call has enough tiles; bf16 and f32 outputs, with the LoRA segment,
    bias and alpha."""
    assert ops.gemm_nt_tile_cols(m, n, k, r) == 384
    assert ops.gemm_nt_tile_cols(512, 384, 4096) == 256          # two tiles: one wave either way
    assert ops.gemm_nt_tile_cols(m, n, 1152, r, torch.float32) == 256      # f32 output under a short K: its epilogue is not overlapped
    g = np.random.Generator(np.random.PCG64(m + n + k))
    a, b = rb(g.standard_normal((m, k))), rb(g.standard_normal((n, k)) * 0.05)
    bias = g.standard_normal(n).astype(np.float32)
    want = a @ b.T                                               # f32 BLAS; compared at bf16 / 1e-4 tolerances below
    kw = {}
    if r:
        a2p = np.zeros((m, 64), np.float32); a2p[:, :r] = rb(g.standard_normal((m, r)))
        b2p = np.zeros((n, 64), np.float32); b2p[:, :r] = rb(g.standard_normal((n, r)))
        want = want + a2p @ b2p.T
        kw = dict(a2=dev(a2p, torch.bfloat16)[:, :r], b2=dev(b2p, torch.bfloat16)[:, :r])
    want = 0.25 * want + bias
    got16 = host(ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16), bias=dev(bias), alpha=0.25, **kw))
    close_bf16(got16, want, rel=6e-3)
    if not r:        # f32 outputs take the K split, which has no second segment
        assert ops.gemm_nt_tile_cols(m, n, k, 0, torch.float32) == 384
        got = host(ops.gemm_nt(dev(a, torch.bfloat16), dev(b, torch.bfloat16), bias=dev(bias), alpha=0.25, out_dtype=torch.float32))
        assert rel_err(got, want) < 1e-4
    assert ops.device_status() == 0


def test_gemm_rejects_bad_arguments(ops):
    from mobilefinetuner_b200._lib import MftError
    a = torch.zeros(8, 12, device="cuda", dtype=torch.bfloat16)   # row stride 12: not a multiple of 8
    b = torch.zeros(8, 12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(MftError):
        ops.gemm_nt(a, b)


@pytest.mark.parametrize("t,p,q", [(64, 8, 8), (1000, 136, 64), (4096, 64, 1536), (777, 1152, 64)])
def test_gemm_tn_acc(ops, t, p, q):
    g = np.random.Generator(np.random.PCG64(t + p + q))
    u, v = rb(g.standard_normal((t, p))), rb(g.standard_normal((t, q)))
    base = g.standard_normal((p, q)).astype(np.float32)
    want = base + 0.25 * (u.astype(np.float64).T @ v.astype(np.float64))
    out = dev(base)
    ops.gemm_tn_acc(dev(u, torch.bfloat16), dev(v, torch.bfloat16), out, alpha=0.25)
    assert rel_err(host(out), want) < 2e-5


@pytest.mark.parametrize("t,p,r,swap", [(2048 + 40, 1152, 16, False), (4096, 6912, 16, True), (1024, 256, 24, False)])
def test_gemm_tn_acc_rank_slice(ops, t, p, r, swap):
    """The LoRA-gradient shape: one operand is the first r columns of a 64-wide buffer (row stride 64).
    P = 6912 takes the tcgen05 kernel (both operands MN-major), the narrower ones the mma.sync kernel."""
    g = np.random.Generator(np.random.PCG64(t + p + r))
    u = rb(g.standard_normal((t, p)))
    wide = rb(g.standard_normal((t, 64)))
    ud, wd = dev(u, torch.bfloat16), dev(wide, torch.bfloat16)
    if swap:
        want = wide[:, :r].astype(np.float64).T @ u.astype(np.float64)
        out = torch.zeros(r, p, device="cuda")
        ops.gemm_tn_acc(wd[:, :r], ud, out)
    else:
        want = u.astype(np.float64).T @ wide[:, :r].astype(np.float64)
        out = torch.zeros(p, r, device="cuda")
        ops.gemm_tn_acc(ud, wd[:, :r], out)
    assert rel_err(host(out), want) < 2e-5
    assert ops.device_status() == 0


def lora_linear_cuda(ops, x, W, bias, A, B, scale, dY):
    """The LoRA-augmented linear as the step composes it: the rank-r update rides in the base
    GEMM as an extra 64-wide k-block (forward and dX); dA/dB are token-contracting TN products."""
    bf = torch.bfloat16
    T, K = x.shape[0] * x.shape[1], x.shape[2]
    N, r = W.shape[1], A.shape[1]
    x2 = dev(x.reshape(T, K), bf)
    Wt = dev(W.T, bf)                 # [N, K]  forward operand (K-major)
    Wn = dev(W, bf)                   # [K, N]  backward operand
    A_nk = torch.zeros(64, K, device="cuda", dtype=bf); A_nk[:r] = dev(A.T, bf)     # [64, K]
    A_kn = torch.zeros(K, 64, device="cuda", dtype=bf); A_kn[:, :r] = dev(A, bf)    # [K, 64]
    B_nk = torch.zeros(N, 64, device="cuda", dtype=bf); B_nk[:, :r] = dev(B.T, bf)  # [N, 64]
    B_kn = torch.zeros(64, N, device="cuda", dtype=bf); B_kn[:r] = dev(B, bf)       # [64, N]
    xa = ops.gemm_nt(x2, A_nk, alpha=scale)                                         # s * x A   [T, 64]
    y = ops.gemm_nt(x2, Wt, a2=xa, b2=B_nk, bias=None if bias is None else dev(bias))
    g = dev(dY.reshape(T, N), bf)
    gb = ops.gemm_nt(g, B_kn, alpha=scale)                                          # s * dY B^T [T, 64]
    dx = ops.gemm_nt(g, Wn, a2=gb, b2=A_kn)
    dA = torch.zeros(K, 64, device="cuda"); ops.gemm_tn_acc(x2, gb, dA)
    dB = torch.zeros(64, N, device="cuda"); ops.gemm_tn_acc(xa, g, dB)
    return host(y).reshape(*x.shape[:2], N), host(dx).reshape(x.shape), host(dA)[:, :r], host(dB)[:r]


def test_lora_linear_golden(ops, golden):
    i, o, p = golden.case("lora_linear")
    y, dx, dA, dB = lora_linear_cuda(ops, i["x"], i["W"], i["bias"], i["A"], i["B"], p["scale"], i["dY"])
    close_bf16(y, o["y"]); close_bf16(dx, o["dx"]); close_bf16(dA, o["dA"]); close_bf16(dB, o["dB"])


def test_lora_linear_model_width(ops):
    g = np.random.Generator(np.random.PCG64(77))
    x = g.standard_normal((2, 160, 1152)).astype(np.float32)
    W = (g.standard_normal((1152, 1536)) * 0.02).astype(np.float32)
    A = (g.uniform(-1, 1, (1152, 16)) / np.sqrt(1152)).astype(np.float32)
    B = (g.standard_normal((16, 1536)) * 0.02).astype(np.float32)
    dY = g.standard_normal((2, 160, 1536)).astype(np.float32)
    y, dx, dA, dB = lora_linear_cuda(ops, x, W, None, A, B, 2.0, dY)
    xr, Wr, Ar, Br, dYr = rb(x), rb(W), rb(A), rb(B), rb(dY)
    want_y = R.lora_linear_fwd(xr, Wr, None, Ar, Br, 2.0)
    want_dx, want_dA, want_dB = R.lora_linear_bwd(xr, Wr, Ar, Br, 2.0, dYr)
    close_bf16(y, want_y); close_bf16(dx, want_dx); close_bf16(dA, want_dA); close_bf16(dB, want_dB)


# ------------------------------------------------------------------ gated MLP fused into the GEMM epilogues
@pytest.mark.parametrize("kind_name,m,inter,k,r,with_bias", [("geglu", 512, 256, 128, 16, False), ("geglu", 300, 384, 200, 0, False),
                                                             ("swiglu", 1024, 4864, 896, 16, True), ("geglu", 768, 6912, 1152, 32, False),
                                                             ("swiglu", 4096, 1536, 640, 16, True)])
def test_fused_gated_mlp_equals_gemm_plus_activation_kernel(ops, kind_name, m, inter, k, r, with_bias):
    """mft_glu_linear_fwd / _bwd (gating inside the CTA-pair GEMM's epilogue) against the same GEMM followed by the
    stand-alone activation kernels, which are pinned to the reference's golden vectors: bit-identical by construction
    (both round gate / up / d_act to bf16 before the gating)."""
    from mobilefinetuner_b200 import _lib as L
    kind = L.ACT_GEGLU if kind_name == "geglu" else L.ACT_SWIGLU
    g = torch.Generator(device="cuda").manual_seed(m + inter + k)
    bf = torch.bfloat16
    x = torch.randn(m, k, device="cuda", generator=g).to(bf)
    w = (torch.randn(2 * inter, k, device="cuda", generator=g) * 0.05).to(bf)
    xa = torch.randn(m, 64, device="cuda", generator=g).to(bf)[:, :r] if r else None
    bp = (torch.randn(2 * inter, 64, device="cuda", generator=g) * 0.05).to(bf)[:, :r] if r else None
    bias = torch.randn(2 * inter, device="cuda", generator=g) * 0.1 if with_bias else None
    fused = ops.glu_linear_fwd(kind, x, w, xa=xa, b_nk=bp, bias=bias)
    assert fused is not None, "the shape qualifies for the fused kernel"
    gu_f, act_f = fused
    gu = ops.gemm_nt(x, w, a2=xa, b2=bp, bias=bias)
    act = ops.act_fwd(kind, gu[:, :inter], gu[:, inter:])
    assert torch.equal(gu_f, gu) and torch.equal(act_f, act)
    # sanity against float64 as well (the activation kernel itself is pinned by the golden tests)
    assert torch.isfinite(act_f.float()).all()
    # backward: dy [m, k'] x down-projection weight [inter, k'] -> d_act, then the gating's backward
    kd = 128 if k < 512 else 640
    dy = torch.randn(m, kd, device="cuda", generator=g).to(bf)
    wd = (torch.randn(inter, kd, device="cuda", generator=g) * 0.05).to(bf)
    a2 = torch.randn(m, 64, device="cuda", generator=g).to(bf)[:, :r] if r else None
    b2 = (torch.randn(inter, 64, device="cuda", generator=g) * 0.05).to(bf)[:, :r] if r else None
    dgu_f = ops.glu_linear_bwd(kind, dy, wd, gu, a2=a2, b2=b2)
    assert dgu_f is not None
    d_act = ops.gemm_nt(dy, wd, a2=a2, b2=b2)
    dg, du = ops.act_bwd(kind, d_act, gu[:, :inter], gu[:, inter:])
    assert torch.equal(dgu_f[:, :inter], dg) and torch.equal(dgu_f[:, inter:], du)
    assert ops.device_status() == 0


def test_fused_gated_mlp_declines_shapes_it_does_not_cover(ops):
    from mobilefinetuner_b200 import _lib as L
    bf = torch.bfloat16
    x = torch.zeros(64, 128, device="cuda", dtype=bf)                     # fewer than 256 rows
    assert ops.glu_linear_fwd(L.ACT_GEGLU, x, torch.zeros(512, 128, device="cuda", dtype=bf)) is None
    x = torch.zeros(512, 128, device="cuda", dtype=bf)                    # inter = 200: not a multiple of 128
    assert ops.glu_linear_fwd(L.ACT_GEGLU, x, torch.zeros(400, 128, device="cuda", dtype=bf)) is None


# ------------------------------------------------------------------ attention
def run_attention(ops, q, k, v, dO, scale, window, theta, split_heads=True):
    bf = torch.bfloat16
    B, nh, S, hd = q.shape
    nkv = k.shape[1]

    def to_dev(x):   # [B,H,S,D] -> token-major storage [B,S,H,D], viewed back as [B,H,S,D]
        return dev(np.ascontiguousarray(x.transpose(0, 2, 1, 3)), bf).permute(0, 2, 1, 3)

    qd, kd, vd, dod = to_dev(q), to_dev(k), to_dev(v), to_dev(dO)
    if theta > 0:
        cos, sin = ops.rope_tables(S, hd, theta, "cuda")
        q_in, k_in = qd, kd
        qd = ops.headnorm_rope_fwd(q_in.permute(0, 2, 1, 3).reshape(B * S, nh * hd), S, nh, hd, cos, sin)[0].view(B, S, nh, hd).permute(0, 2, 1, 3)
        kd = ops.headnorm_rope_fwd(k_in.permute(0, 2, 1, 3).reshape(B * S, nkv * hd), S, nkv, hd, cos, sin)[0].view(B, S, nkv, hd).permute(0, 2, 1, 3)
    o, lse = ops.attention_fwd(qd, kd, vd, scale, window)
    dq, dk, dv = ops.attention_bwd(qd, kd, vd, o, dod, lse, scale, window, split_heads=split_heads)
    if theta > 0:
        dq = ops.headnorm_rope_bwd(dq.permute(0, 2, 1, 3).reshape(B * S, nh * hd), None, S, nh, hd, cos, sin).view(B, S, nh, hd).permute(0, 2, 1, 3)
        dk = ops.headnorm_rope_bwd(dk.permute(0, 2, 1, 3).reshape(B * S, nkv * hd), None, S, nkv, hd, cos, sin).view(B, S, nkv, hd).permute(0, 2, 1, 3)
    return host(o), host(dq), host(dk), host(dv)


@pytest.mark.parametrize("split_heads", [True, False])
@pytest.mark.parametrize("name", ["attn_causal_gqa", "attn_window_rope", "attn_hd256_window", "attn_hd128"])
def test_attention_golden(ops, golden, name, split_heads):
    i, o, p = golden.case(name)
    out, dq, dk, dv = run_attention(ops, i["q"], i["k"], i["v"], i["dO"], p["scale"], int(p["window"]), p["rope_theta"], split_heads)
    close_bf16(out, o["O"]); close_bf16(dq, o["dQ"]); close_bf16(dk, o["dK"]); close_bf16(dv, o["dV"])


@pytest.mark.parametrize("S", [256, 512])
def test_attention_operator_sweep_shapes(ops, S):
    """The operator-level benchmark shape: batch 8, 14 query heads, 2 KV heads, head_dim 64, N(0,1) inputs."""
    g = np.random.Generator(np.random.PCG64(4000 + S))
    B, nh, nkv, hd = 8, 14, 2, 64
    q, k, v, dO = (rb(g.standard_normal(s)) for s in [(B, nh, S, hd), (B, nkv, S, hd), (B, nkv, S, hd), (B, nh, S, hd)])
    out, dq, dk, dv = run_attention(ops, q, k, v, dO, 0.125, 0, 0.0)
    w_out, w_dq, w_dk, w_dv = R.attention_fwd_bwd(q, k, v, dO, 0.125)
    close_bf16(out, w_out); close_bf16(dq, w_dq); close_bf16(dk, w_dk); close_bf16(dv, w_dv)


def test_attention_mask_predicate_is_exact(ops):
    """With V = one-hot rows the output reveals exactly which keys were visible: the causal /
    sliding-window pattern must equal the reference predicate (j <= i and i - j < window)."""
    B, nh, S, hd, window = 1, 1, 200, 256, 37
    q = np.zeros((B, nh, S, hd), np.float32)
    k = np.zeros((B, nh, S, hd), np.float32)
    v = np.zeros((B, nh, S, hd), np.float32)
    for j in range(S):
        v[0, 0, j, j] = 1.0        # S <= hd: column j marks key j
    out, *_ = run_attention(ops, q, k, v, np.zeros_like(q), 1.0, window, 0.0)
    visible = out[0, 0, :, :S] > 0
    i, j = np.arange(S)[:, None], np.arange(S)[None, :]
    assert np.array_equal(visible, (j <= i) & (i - j < window))


@pytest.mark.parametrize("S,window,nkv,amp", [(128, 0, 1, 1.0), (384, 0, 2, 1.0), (512, 200, 1, 1.0), (256, 64, 4, 1.0), (384, 0, 1, 6.0)])
def test_attention_head_dim_256_tensor_memory_path(ops, S, window, nkv, amp):
    """head_dim 256 with a sequence that is a multiple of 128 runs on the tcgen05 kernels (scores and output
    accumulator in tensor memory).  amp > 1 makes the row maxima grow quickly along the keys, which exercises the
    rescale of the accumulator."""
    g = np.random.Generator(np.random.PCG64(9000 + S + window))
    B, nh, hd = 2, 4, 256
    q, dO = rb(g.standard_normal((B, nh, S, hd)) * amp), rb(g.standard_normal((B, nh, S, hd)))
    k, v = rb(g.standard_normal((B, nkv, S, hd)) * amp), rb(g.standard_normal((B, nkv, S, hd)))
    if amp > 1.0:
        k = rb(k * np.linspace(0.2, 1.0, S, dtype=np.float32)[None, None, :, None])    # later keys score higher
    out, dq, dk, dv = run_attention(ops, q, k, v, dO, hd ** -0.5, window, 0.0)
    w_out, w_dq, w_dk, w_dv = R.attention_fwd_bwd(q, k, v, dO, hd ** -0.5, window)
    close_bf16(out, w_out); close_bf16(dq, w_dq); close_bf16(dk, w_dk); close_bf16(dv, w_dv)
    assert ops.device_status() == 0


def test_attention_full_size_properties(ops):
    """S = 4096 (too large for the dense CPU chain): uniform-attention identity.  With Q = 0 every
    visible key gets the same weight, so O[i] is the running mean of V and dV[j] = sum_{i>=j} dO[i]/(i+1)."""
    B, nh, nkv, S, hd = 1, 2, 1, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.zeros(B, S, nh, hd, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    k = torch.randn(B, S, nkv, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    v = torch.randn(B, S, nkv, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    o, lse = ops.attention_fwd(q, k, v, 0.125, 0)
    want = torch.cumsum(v.float(), dim=2) / torch.arange(1, S + 1, device="cuda").view(1, 1, S, 1)
    assert (o.float() - want.expand(B, nh, S, hd)).abs().max().item() < 2e-2
    assert torch.allclose(lse, torch.log(torch.arange(1, S + 1, device="cuda").float()).expand(B, nh, S), atol=1e-3)


@pytest.mark.parametrize("window", [0, 512])
def test_attention_head_dim_256_full_size_properties(ops, window):
    """The headline shape (S = 2048, head_dim 256, 4 query heads on 1 KV head) on the tensor-memory kernels, checked
    through the uniform-attention identity: with Q = 0 every visible key has the same weight, so O[i] is the mean of
    the visible V rows, lse[i] = log(#visible), dV[j] = sum over the queries that see j of dO[i] / #visible(i),
    and dQ = scale * (P (dP - delta)) K with dP - delta = dO[i] . (V[j] - O[i])."""
    B, nh, nkv, S, hd = 1, 4, 1, 2048, 256
    g = torch.Generator(device="cuda").manual_seed(7)
    q = torch.zeros(B, S, nh, hd, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    k = torch.randn(B, S, nkv, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    v = torch.randn(B, S, nkv, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    do = torch.randn(B, S, nh, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    scale = hd ** -0.5
    o, lse = ops.attention_fwd(q, k, v, scale, window)
    i = torch.arange(S, device="cuda")
    vis = (i[None, :] <= i[:, None]) & ((i[:, None] - i[None, :] < window) if window > 0 else torch.ones(S, S, dtype=torch.bool, device="cuda"))
    cnt = vis.sum(1).double()                                            # visible keys per query
    P = vis.double() / cnt[:, None]
    want_o = (P @ v[0, 0].double())                                      # [S, hd], same for every head
    assert (o.double() - want_o[None, None]).abs().max().item() < 2e-2
    assert torch.allclose(lse.double(), torch.log(cnt).expand(B, nh, S), atol=1e-3)
    dq, dk, dv = ops.attention_bwd(q, k, v, o, do, lse, scale, window)
    want_dv = sum(P.T @ do[0, h].double() for h in range(nh))            # [S, hd]
    assert cosine(host(dv[0, 0].float()), want_dv.cpu().numpy()) >= 0.9995
    dP = do[0, 0].double() @ v[0, 0].double().T                          # head 0
    delta = (do[0, 0].double() * o[0, 0].double()).sum(1, keepdim=True)
    want_dq0 = scale * ((P * (dP - delta)) @ k[0, 0].double())
    assert cosine(host(dq[0, 0].float()), want_dq0.cpu().numpy()) >= 0.9995
    assert ops.device_status() == 0


# ------------------------------------------------------------------ norms, activations, RoPE, gathers
@pytest.mark.parametrize("dim", [640, 1152, 2048])
def test_fused_norm_pairs_equal_the_separate_kernels(ops, dim):
    """Gemma's post-norm + residual add + next pre-norm in one kernel, forward and backward: bit-identical to the
    separate rms_norm kernels (which are pinned to the reference's golden vectors)."""
    g = torch.Generator(device="cuda").manual_seed(dim)
    rows, eps = 300, 1e-6
    y = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    x = torch.randn(rows, dim, device="cuda", generator=g)
    wp = torch.randn(dim, device="cuda", generator=g) * 0.1
    wn = torch.randn(dim, device="cuda", generator=g) * 0.1
    _, rp_ref, sum_ref = ops.rms_norm_fwd(y, wp, eps, 1, out_dtype=torch.bfloat16, residual=x)
    h_ref, rn_ref = ops.rms_norm_fwd(sum_ref, wn, eps, 1, out_dtype=torch.bfloat16)
    s, rp, h, rn = ops.rms_norm_add_norm_fwd(y, wp, x, wn, eps)
    assert torch.equal(s, sum_ref) and torch.equal(rp, rp_ref) and torch.equal(h, h_ref) and torch.equal(rn, rn_ref)
    dy = torch.randn(rows, dim, device="cuda", generator=g).bfloat16()
    dx0 = torch.randn(rows, dim, device="cuda", generator=g)
    dx_ref = ops.rms_norm_bwd(dy, sum_ref, wn, rn_ref, eps, 1, accumulate_into=dx0.clone())
    db_ref = ops.rms_norm_bwd(dx_ref, y, wp, rp_ref, eps, 1, out_dtype=torch.bfloat16)
    dx = dx0.clone()
    db = ops.rms_norm_pair_bwd(dy, s, wn, rn, dx, y, wp, rp)
    assert torch.equal(dx, dx_ref) and torch.equal(db, db_ref)


@pytest.mark.parametrize("name,unit", [("rms_norm", 1), ("rms_norm_affine", 0)])
def test_rms_norm_golden_fp32(ops, golden, name, unit):
    i, o, p = golden.case(name)
    x, w, dy = dev(i["x"]), dev(i["w"]), dev(i["dY"])
    y, rstd = ops.rms_norm_fwd(x, w, p["eps"], unit, out_dtype=torch.float32)
    assert rel_err(host(y), o["y"]) < 1e-5
    dw = torch.zeros_like(w)
    dx = ops.rms_norm_bwd(dy, x, w, rstd, p["eps"], unit, dweight=dw)
    assert rel_err(host(dx), o["dx"]) < 1e-5 and rel_err(host(dw), o["dw"]) < 1e-5


def test_rms_norm_fused_residual_and_bf16(ops):
    g = np.random.Generator(np.random.PCG64(3))
    x, res, w = g.standard_normal((300, 1152)).astype(np.float32), g.standard_normal((300, 1152)).astype(np.float32), (g.standard_normal(1152) * 0.1).astype(np.float32)
    y, rstd, s = ops.rms_norm_fwd(dev(rb(x), torch.bfloat16), dev(w), 1e-6, 1, out_dtype=torch.bfloat16, residual=dev(res))
    want = R.rms_norm_fwd(rb(x), w, 1e-6, True)
    close_bf16(host(y), want, rel=8e-3)
    assert rel_err(host(s), want + res) < 1e-5 * 50


def test_layer_norm_golden(ops, golden):
    i, o, p = golden.case("layer_norm")
    x, w, b, dy = dev(i["x"]), dev(i["w"]), dev(i["b"]), dev(i["dY"])
    y, mean, rstd = ops.layer_norm_fwd(x, w, b, p["eps"], out_dtype=torch.float32)
    assert rel_err(host(y), o["y"]) < 1e-5
    dw, db = torch.zeros_like(w), torch.zeros_like(b)
    dx = ops.layer_norm_bwd(dy, x, w, mean, rstd, dweight=dw, dbias=db)
    assert rel_err(host(dx), o["dx"]) < 5e-5 and rel_err(host(dw), o["dw"]) < 1e-5 and rel_err(host(db), o["db"]) < 1e-5


@pytest.mark.parametrize("name,kind", [("gelu", 0), ("swiglu", 1), ("geglu", 2)])
def test_activations_golden(ops, golden, name, kind):
    i, o, _ = golden.case(name)
    bf = torch.bfloat16
    gate = i["x"] if name == "gelu" else i["gate"]
    up = None if name == "gelu" else i["up"]
    g2 = dev(gate.reshape(-1, gate.shape[-1]), bf)
    u2 = None if up is None else dev(up.reshape(-1, up.shape[-1]), bf)
    dy = dev(i["dY"].reshape(-1, gate.shape[-1]), bf)
    y = ops.act_fwd(kind, g2, u2)
    dg, du = ops.act_bwd(kind, dy, g2, u2)
    close_bf16(host(y).reshape(gate.shape), o["y"], rel=1e-2)
    close_bf16(host(dg).reshape(gate.shape), o["dx" if name == "gelu" else "dgate"], rel=1.5e-2)
    if up is not None:
        close_bf16(host(du).reshape(gate.shape), o["dup"], rel=1.5e-2)


@pytest.mark.parametrize("name", ["rope_1e4", "rope_1e6"])
def test_rope_golden_and_table_bits(ops, golden, name):
    i, o, p = golden.case(name)
    B, H, S, hd = i["x"].shape
    cos, sin = ops.rope_tables(S, hd, p["rope_theta"], "cuda")
    rc, rs = R.rope_tables(S, hd, p["rope_theta"])
    # angles are computed on the host with the reference's own float expression (libm powf/cosf/sinf);
    # numpy's float32 power differs from libm by an ulp, hence a few 1e-6 at angles of tens of radians
    assert np.abs(host(cos) - rc).max() < 1e-5 and np.abs(host(sin) - rs).max() < 1e-5
    x = dev(np.ascontiguousarray(i["x"].transpose(0, 2, 1, 3)).reshape(B * S, H * hd), torch.bfloat16)
    y, _ = ops.headnorm_rope_fwd(x, S, H, hd, cos, sin)
    close_bf16(host(y).reshape(B, S, H, hd).transpose(0, 2, 1, 3), o["y"], rel=1e-2)
    dy = dev(np.ascontiguousarray(i["dY"].transpose(0, 2, 1, 3)).reshape(B * S, H * hd), torch.bfloat16)
    dx = ops.headnorm_rope_bwd(dy, None, S, H, hd, cos, sin)
    close_bf16(host(dx).reshape(B, S, H, hd).transpose(0, 2, 1, 3), o["dx"], rel=1e-2)


def test_headnorm_rope_matches_norm_then_rope(ops):
    """Gemma applies rms_norm(1+w) per head, then RoPE (gemma_model.cpp:459-482)."""
    g = np.random.Generator(np.random.PCG64(9))
    B, S, H, hd = 2, 50, 4, 256
    x = rb(g.standard_normal((B, H, S, hd)))
    w = (g.standard_normal(hd) * 0.1).astype(np.float32)
    dy = rb(g.standard_normal((B, H, S, hd)))
    want = R.rope_fwd(R.rms_norm_fwd(x, w, 1e-6, True), 10000.0)
    want_dx, _ = R.rms_norm_bwd(R.rope_bwd(dy, 10000.0), x, w, 1e-6, True)
    cos, sin = ops.rope_tables(S, hd, 10000.0, "cuda")
    xt = dev(np.ascontiguousarray(x.transpose(0, 2, 1, 3)).reshape(B * S, H * hd), torch.bfloat16)
    y, rstd = ops.headnorm_rope_fwd(xt, S, H, hd, cos, sin, norm_weight=dev(w), eps=1e-6)
    close_bf16(host(y).reshape(B, S, H, hd).transpose(0, 2, 1, 3), want, rel=1e-2)
    dyt = dev(np.ascontiguousarray(dy.transpose(0, 2, 1, 3)).reshape(B * S, H * hd), torch.bfloat16)
    dx = ops.headnorm_rope_bwd(dyt, xt, S, H, hd, cos, sin, norm_weight=dev(w), rstd=rstd)
    close_bf16(host(dx).reshape(B, S, H, hd).transpose(0, 2, 1, 3), want_dx, rel=1.5e-2)


def test_repeat_kv_bit_exact(ops, golden):
    i, o, p = golden.case("repeat_kv")
    rep = int(p["repeat"])
    assert np.array_equal(host(ops.repeat_kv(dev(i["x"]), rep)), o["y"])
    assert rel_err(host(ops.repeat_kv_bwd(dev(i["dY"]), rep)), o["dx"]) < 1e-6


def test_embedding_gather_bit_exact(ops):
    g = np.random.Generator(np.random.PCG64(21))
    V, H, B, S = 1000, 640, 3, 17
    table = rb(g.standard_normal((V, H)) * 0.02)
    ids = g.integers(0, V, size=(B, S)).astype(np.int32)
    got = host(ops.embedding_gather(dev(ids), dev(table, torch.bfloat16), 1.0))
    assert np.array_equal(got, table[ids.ravel()])             # pure gather: exact bits
    scale = np.float32(np.sqrt(np.float32(H)))
    got = host(ops.embedding_gather(dev(ids), dev(table, torch.bfloat16), float(scale)))
    assert np.array_equal(got, table[ids.ravel()] * scale)
    pos = rb(g.standard_normal((32, H)) * 0.02)
    got = host(ops.embedding_gather(dev(ids), dev(table, torch.bfloat16), 1.0, dev(pos, torch.bfloat16), S))
    assert np.array_equal(got.reshape(B, S, H), table[ids] + pos[:S][None])
    ids[1, 2] = V
    with pytest.raises(IndexError):
        ops.embedding_gather(dev(ids), dev(table, torch.bfloat16), 1.0)


# ------------------------------------------------------------------ loss
def test_lm_head_ce_golden(ops, golden):
    i, o, _ = golden.case("lm_head_ce")
    ce = ops.LmHeadCE(dev(i["W"], torch.bfloat16))
    hid = dev(i["hidden"], torch.bfloat16)
    labels = dev(i["labels"])
    loss = ce.forward(hid, labels)
    assert int(ce.n_valid.item()) == int((i["labels"][:, 1:] != -100).sum())   # integer work: exact
    assert abs(loss.item() - o["loss"][0]) <= 2e-3 * abs(o["loss"][0])
    dh = ce.backward(hid, labels)
    close_bf16(host(dh), o["dhidden"])
    assert ops.device_status() == 0


def test_lm_head_ce_large_vocab_vs_restatement(ops, ce_panels):
    g = np.random.Generator(np.random.PCG64(31))
    B, S, H, V = 2, 70, 640, 20000          # several vocabulary panels, ragged last tile
    hid = rb(g.standard_normal((B, S, H)))
    W = rb(g.standard_normal((V, H)) * 0.05)
    labels = g.integers(0, V, size=(B, S)).astype(np.int32)
    labels[0, 5:9] = -100
    want_loss, want_dh = R.lm_head_ce(hid, W, labels)
    ce = ops.LmHeadCE(dev(W, torch.bfloat16))
    loss = ce.forward(dev(hid, torch.bfloat16), dev(labels))
    assert abs(loss.item() - want_loss) <= 2e-3 * abs(want_loss)
    dh = host(ce.backward(dev(hid, torch.bfloat16), dev(labels)))
    close_bf16(dh, want_dh)
    assert np.all(dh[:, -1, :] == 0) and np.all(dh[0, 4:8, :] == 0)    # unscored rows get exactly zero


def test_lm_head_ce_fused_golden_and_two_sweep(ops, golden):
    """One sweep over the vocabulary gives the loss and dHidden of the forward + backward pair."""
    i, o, _ = golden.case("lm_head_ce")
    ce = ops.LmHeadCE(dev(i["W"], torch.bfloat16))
    hid, labels = dev(i["hidden"], torch.bfloat16), dev(i["labels"])
    loss, dh = ce.fused(hid, labels)
    assert int(ce.n_valid.item()) == int((i["labels"][:, 1:] != -100).sum())
    assert abs(loss.item() - o["loss"][0]) <= 2e-3 * abs(o["loss"][0])
    close_bf16(host(dh), o["dhidden"])
    lse1 = host(ce.lse).copy()
    ce.forward(hid, labels)
    np.testing.assert_allclose(lse1, host(ce.lse), rtol=0, atol=2e-3)
    assert ops.device_status() == 0


@pytest.fixture(params=["whole vocabulary", "8192-column panels"])
def ce_panels(request):
    """The lm-head loss walks the vocabulary in panels; by default one panel covers it when the buffer fits."""
    from mobilefinetuner_b200 import _lib as L
    old = L.call("mft_lmhead_ce_set_panel_budget", 1 if request.param != "whole vocabulary" else 12 << 30)
    yield request.param
    L.call("mft_lmhead_ce_set_panel_budget", old)


def test_lm_head_ce_fused_large_vocab_dp_scaling(ops, ce_panels):
    g = np.random.Generator(np.random.PCG64(32))
    B, S, H, V = 2, 70, 640, 20000
    hid = rb(g.standard_normal((B, S, H)))
    W = rb(g.standard_normal((V, H)) * 0.05)
    labels = g.integers(0, V, size=(B, S)).astype(np.int32)
    labels[1, 10:20] = -100
    want_loss, want_dh = R.lm_head_ce(hid, W, labels)
    ce = ops.LmHeadCE(dev(W, torch.bfloat16))
    loss, dh = ce.fused(dev(hid, torch.bfloat16), dev(labels))
    assert abs(loss.item() - want_loss) <= 2e-3 * abs(want_loss)
    dh = host(dh)
    close_bf16(dh, want_dh)
    assert np.all(dh[:, -1, :] == 0) and np.all(dh[1, 9:19, :] == 0)
    n = int(ce.n_valid.item())
    _, dh2 = ce.fused(dev(hid, torch.bfloat16), dev(labels), n_valid_override=2 * n)   # a data-parallel rank: global count
    close_bf16(host(dh2), want_dh / 2)


def test_lm_head_ce_fused_recomputes_rows_out_of_range(ops, ce_panels):
    """Logits far above the first panel's log-sum-exp: the sweep flags those rows and recomputes them exactly."""
    g = np.random.Generator(np.random.PCG64(33))
    B, S, H, V = 1, 40, 128, 16384 + 300       # second panel holds the large logits
    hid = rb(g.standard_normal((B, S, H)))
    W = rb(g.standard_normal((V, H)) * 0.05)
    for r in range(0, S, 3):                   # every third row points at its own column of panel 2
        W[16384 + r] = rb(hid[0, r] * (150.0 / float(hid[0, r] @ hid[0, r])))
    labels = g.integers(0, V, size=(B, S)).astype(np.int32)
    labels[0, 4] = 16384 + 3
    want_loss, want_dh = R.lm_head_ce(hid, W, labels)
    ce = ops.LmHeadCE(dev(W, torch.bfloat16))
    loss, dh = ce.fused(dev(hid, torch.bfloat16), dev(labels))
    assert np.isfinite(loss.item()) and abs(loss.item() - want_loss) <= 2e-3 * abs(want_loss)
    close_bf16(host(dh), want_dh)
    ce.forward(dev(hid, torch.bfloat16), dev(labels))
    assert abs(loss.item() - ce.loss.item()) <= 1e-3 * abs(want_loss)


def test_lm_ce_all_ignored_and_out_of_range(ops, golden):
    i, o, _ = golden.case("lm_ce_all_ignored")
    ce = ops.LmHeadCE(dev(i["W"], torch.bfloat16))
    hid, labels = dev(i["hidden"], torch.bfloat16), dev(i["labels"])
    assert np.isnan(ce.forward(hid, labels).item()) and np.isnan(o["loss"][0])
    assert np.all(host(ce.backward(hid, labels)) == 0)
    loss, dh = ce.fused(hid, labels)
    assert np.isnan(loss.item()) and np.all(host(dh) == 0)
    bad = i["labels"].copy(); bad[0, 3] = i["W"].shape[0]
    with pytest.raises(IndexError):
        ce.forward(hid, dev(bad))


def test_ce_dense_golden(ops, golden):
    i, o, _ = golden.case("lm_ce")
    loss, dlogits = ops.ce_dense(dev(i["logits"]), dev(i["labels"]))
    assert abs(loss.item() - o["loss"][0]) < 1e-5 * abs(o["loss"][0])
    assert rel_err(host(dlogits), o["dlogits"]) < 1e-5


# ------------------------------------------------------------------ optimizer
@pytest.mark.parametrize("name", ["adam_clip", "adam_wd"])
def test_adam_golden(ops, golden, name):
    i, o, p = golden.case(name)
    params = dev(i["p"].ravel().copy())
    m, v = torch.zeros_like(params), torch.zeros_like(params)
    for step in range(int(p["steps"])):
        grads = dev(i[f"g{step}"].ravel().copy())
        ops.adam_step(params, grads, m, v, step + 1, p["lr"], weight_decay=p.get("weight_decay", 0.0),
                      max_norm=p.get("max_grad_norm", 0.0), clip_eps=0.0, zero_grad=True)
        assert float(grads.abs().max()) == 0.0
    assert rel_err(host(params), o["p"].ravel()) < 2e-6
