"""Single-kernel microbenchmarks (CUDA-event timing) for the kernels of the LoRA step.

    python -m mobilefinetuner_b200.microbench gemm --m 4096 --n 13824 --k 1152 [--k2 32] [--f32] [--iters 20]
    python -m mobilefinetuner_b200.microbench glu --m 16384 --n 6912 --k 1152 --k2 16      # gated MLP: fused launches against GEMM + activation
    python -m mobilefinetuner_b200.microbench attn --batch 8 --heads 4 --kv-heads 1 --seq 2048 --head-dim 256 [--window 512]
    python -m mobilefinetuner_b200.microbench tn --t 16384 --p 1152 --q 64
    python -m mobilefinetuner_b200.microbench ce --t 4096 --hidden 1152 --vocab 262144
    python -m mobilefinetuner_b200.microbench tma                                          # L2 -> shared memory delivery per SM (no MMAs)

Prints one JSON line per run with the achieved TFLOP/s or GB/s; the same command under a profiler
captures just that kernel.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops as O

BF = torch.bfloat16


def _time(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemm", "glu", "attn", "tn", "ce", "tma"])
    ap.add_argument("--no-split", action="store_true", help="attn: one CTA per KV group in the dK/dV kernel")
    ap.add_argument("--m", type=int, default=16384); ap.add_argument("--n", type=int, default=13824); ap.add_argument("--k", type=int, default=1152)
    ap.add_argument("--k2", type=int, default=0); ap.add_argument("--f32", action="store_true")
    ap.add_argument("--batch", type=int, default=8); ap.add_argument("--heads", type=int, default=4); ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--seq", type=int, default=2048); ap.add_argument("--head-dim", type=int, default=256); ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--t", type=int, default=16384); ap.add_argument("--p", type=int, default=1152); ap.add_argument("--q", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=1152); ap.add_argument("--vocab", type=int, default=262144)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    out = {"kind": a.kind}
    if a.kind == "tma":
        # one JSON line per (SMs pulling, load kind, stages in flight)
        import ctypes as C
        from . import _lib as L
        L.init(torch.cuda.current_device())
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        names = {0: "two 128-row tensor boxes per stage", 1: "two 16 KB bulk copies per stage", 2: "one box and one bulk copy per stage"}
        for ctas, mode, stages in [(sms, 0, 6), (sms, 1, 6), (sms, 2, 6), (sms // 2, 0, 6), (16, 0, 6), (sms, 0, 1), (sms, 0, 2), (sms, 0, 3), (sms, 0, 4)]:
            bpc, tbs = C.c_double(), C.c_double()
            L.call("mft_probe_tma_delivery", mode, stages, ctas, 4000, C.byref(bpc), C.byref(tbs), None)
            print(json.dumps({"kind": "tma", "ctas": ctas, "loads": names[mode], "stages": stages, "bytes_per_clock_per_sm": round(bpc.value, 1),
                              "tb_per_s": round(tbs.value, 2)}), flush=True)
        return
    if a.kind == "gemm":
        A = torch.randn(a.m, a.k, device=dev, generator=g).to(BF)
        B = torch.randn(a.n, a.k, device=dev, generator=g).to(BF)
        A2 = torch.randn(a.m, 64, device=dev, generator=g).to(BF)[:, :a.k2] if a.k2 else None
        B2 = torch.randn(a.n, 64, device=dev, generator=g).to(BF)[:, :a.k2] if a.k2 else None
        D = torch.empty(a.m, a.n, device=dev, dtype=torch.float32 if a.f32 else BF)
        ms = _time(lambda: O.gemm_nt(A, B, a2=A2, b2=B2, out=D), a.iters)
        fl = 2.0 * a.m * a.n * (a.k + a.k2)
        out.update(m=a.m, n=a.n, k=a.k, k2=a.k2, ms=ms, tflops=fl / ms / 1e9)
    elif a.kind == "glu":
        # gated MLP around the down projection: --n is the intermediate width, --k the hidden width, --k2 the LoRA rank
        # columns of each projection.  Fused launches against GEMM + stand-alone activation kernel.
        from . import _lib as L
        M, I, K, r = a.m, a.n, a.k, a.k2
        kind = L.ACT_GEGLU
        x = torch.randn(M, K, device=dev, generator=g).to(BF)
        w = (torch.randn(2 * I, K, device=dev, generator=g) * 0.05).to(BF)
        xa = torch.randn(M, 64, device=dev, generator=g).to(BF)[:, :2 * r] if r else None
        bp = (torch.randn(2 * I, 64, device=dev, generator=g) * 0.05).to(BF)[:, :2 * r] if r else None
        gu = O.gemm_nt(x, w, a2=xa, b2=bp)
        dy = torch.randn(M, K, device=dev, generator=g).to(BF)
        wd = (torch.randn(I, K, device=dev, generator=g) * 0.05).to(BF)
        a2 = torch.randn(M, 64, device=dev, generator=g).to(BF)[:, :r] if r else None
        b2 = (torch.randn(I, 64, device=dev, generator=g) * 0.05).to(BF)[:, :r] if r else None
        d_act = O.gemm_nt(dy, wd, a2=a2, b2=b2)
        out.update(m=M, inter=I, k=K, k2=r,
                   fwd_fused_ms=_time(lambda: O.glu_linear_fwd(kind, x, w, xa=xa, b_nk=bp), a.iters),
                   fwd_gemm_ms=_time(lambda: O.gemm_nt(x, w, a2=xa, b2=bp), a.iters),
                   fwd_act_ms=_time(lambda: O.act_fwd(kind, gu[:, :I], gu[:, I:]), a.iters),
                   bwd_fused_ms=_time(lambda: O.glu_linear_bwd(kind, dy, wd, gu, a2=a2, b2=b2), a.iters),
                   bwd_gemm_ms=_time(lambda: O.gemm_nt(dy, wd, a2=a2, b2=b2), a.iters),
                   bwd_act_ms=_time(lambda: O.act_bwd(kind, d_act, gu[:, :I], gu[:, I:]), a.iters))
    elif a.kind == "attn":
        b, nh, nkv, s, hd = a.batch, a.heads, a.kv_heads, a.seq, a.head_dim
        q = torch.randn(b, s, nh, hd, device=dev, generator=g).to(BF).permute(0, 2, 1, 3)
        k = torch.randn(b, s, nkv, hd, device=dev, generator=g).to(BF).permute(0, 2, 1, 3)
        v = torch.randn(b, s, nkv, hd, device=dev, generator=g).to(BF).permute(0, 2, 1, 3)
        do = torch.randn(b, s, nh, hd, device=dev, generator=g).to(BF).permute(0, 2, 1, 3)
        scale = hd ** -0.5
        o, lse = O.attention_fwd(q, k, v, scale, a.window)
        ms_f = _time(lambda: O.attention_fwd(q, k, v, scale, a.window), a.iters)
        ms_b = _time(lambda: O.attention_bwd(q, k, v, o, do, lse, scale, a.window, split_heads=not a.no_split), a.iters)
        pairs = sum(min(i + 1, a.window) if a.window > 0 else i + 1 for i in range(s)) * b * nh
        out.update(batch=b, heads=nh, kv_heads=nkv, seq=s, head_dim=hd, window=a.window, fwd_ms=ms_f, bwd_ms=ms_b,
                   fwd_tflops=4.0 * hd * pairs / ms_f / 1e9, bwd_tflops=8.0 * hd * pairs / ms_b / 1e9)
    elif a.kind == "tn":
        U = torch.randn(a.t, a.p, device=dev, generator=g).to(BF)
        V = torch.randn(a.t, a.q, device=dev, generator=g).to(BF)
        out_t = torch.zeros(a.p, a.q, device=dev)
        ms = _time(lambda: O.gemm_tn_acc(U, V, out_t), a.iters)
        out.update(t=a.t, p=a.p, q=a.q, ms=ms, gbs=2.0 * a.t * (a.p + a.q) / ms / 1e6)
    else:
        W = (torch.randn(a.vocab, a.hidden, device=dev, generator=g) * 0.02).to(BF)
        hid = torch.randn(1, a.t, a.hidden, device=dev, generator=g).to(BF)
        labels = torch.randint(0, a.vocab, (1, a.t), device=dev, dtype=torch.int32)
        ce = O.LmHeadCE(W)
        ms_f = _time(lambda: ce.forward(hid, labels), max(2, a.iters // 4))
        ms_b = _time(lambda: ce.backward(hid, labels), max(2, a.iters // 4))
        fl = 2.0 * a.t * a.hidden * a.vocab
        out.update(t=a.t, hidden=a.hidden, vocab=a.vocab, fwd_ms=ms_f, bwd_ms=ms_b, fwd_tflops=fl / ms_f / 1e9,
                   bwd_tflops_algorithmic=fl / ms_b / 1e9, bwd_tflops_executed=2 * fl / ms_b / 1e9)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
