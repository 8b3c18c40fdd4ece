"""Generates tests/golden/ops_golden.npz by running the compiled, unmodified reference
(oracle/_ref/ref_driver_*, built by `make -C oracle` where the reference is mounted) on
small seeded inputs.  Inputs and the reference's outputs are both stored, so the
fixtures are self-contained: the CPU suite pins oracle/restate.py against them and
the GPU suite pins the CUDA kernels against them.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import sys
import zlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import refrun  # noqa: E402

f32 = np.float32


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def normal(g, shape, std=1.0):
    return (g.standard_normal(shape) * std).astype(f32)


def main():
    store = {}

    def put(case, tensors, outputs, **params):
        for k, v in tensors.items():
            store[f"{case}/in/{k}"] = v
        for k, v in outputs.items():
            if not k.startswith("_"):
                store[f"{case}/out/{k}"] = v
        for k, v in params.items():
            store[f"{case}/param/{k}"] = np.asarray(v)

    # attention chain: (name, B, nh, nkv, S, hd, window, theta)
    for name, B, nh, nkv, S, hd, window, theta in [
        ("attn_causal_gqa", 2, 4, 2, 96, 64, 0, 0.0),
        ("attn_window_rope", 1, 4, 1, 80, 64, 24, 10000.0),
        ("attn_hd256_window", 1, 4, 1, 72, 256, 40, 0.0),
        ("attn_hd128", 1, 2, 2, 33, 128, 0, 1000000.0),
    ]:
        g = rng(zlib.crc32(name.encode()))
        t = {"q": normal(g, (B, nh, S, hd)), "k": normal(g, (B, nkv, S, hd)), "v": normal(g, (B, nkv, S, hd)),
             "dO": normal(g, (B, nh, S, hd))}
        scale = 1.0 / np.sqrt(hd)
        out = refrun.run_op("attention", t, scale=scale, window=window, rope_theta=theta)
        put(name, t, out, scale=scale, window=window, rope_theta=theta)

    g = rng(11)
    t = {"x": normal(g, (2, 24, 64)), "W": normal(g, (64, 96), 0.05), "bias": normal(g, (96,), 0.1),
         "A": normal(g, (64, 8), 0.1), "B": normal(g, (8, 96), 0.1), "dY": normal(g, (2, 24, 96))}
    put("lora_linear", t, refrun.run_op("lora_linear", t, scale=2.0), scale=2.0)

    g = rng(12)
    t = {"a": normal(g, (3, 20, 48)), "b": normal(g, (48, 40)), "dY": normal(g, (3, 20, 40))}
    put("matmul", t, refrun.run_op("matmul", t))
    t = {"a": normal(g, (3, 20, 48)), "b": normal(g, (40, 48)), "dY": normal(g, (3, 20, 40))}
    put("matmul_rhs_T", t, refrun.run_op("matmul_rhs_T", t))

    for op in ("rms_norm", "rms_norm_affine"):
        g = rng(13)
        t = {"x": normal(g, (3, 17, 64)), "w": normal(g, (64,), 0.2), "dY": normal(g, (3, 17, 64))}
        put(op, t, refrun.run_op(op, t, eps=1e-6), eps=1e-6)
    g = rng(14)
    t = {"x": normal(g, (5, 9, 128)), "w": (1 + normal(g, (128,), 0.1)).astype(f32), "b": normal(g, (128,), 0.1),
         "dY": normal(g, (5, 9, 128))}
    put("layer_norm", t, refrun.run_op("layer_norm", t, eps=1e-5), eps=1e-5)

    g = rng(15)
    t = {"x": normal(g, (4, 33, 16), 2.0), "dY": normal(g, (4, 33, 16))}
    put("gelu", t, refrun.run_op("gelu", t))
    for op in ("swiglu", "geglu"):
        t = {"gate": normal(g, (4, 33, 16), 2.0), "up": normal(g, (4, 33, 16)), "dY": normal(g, (4, 33, 16))}
        put(op, t, refrun.run_op(op, t))

    for name, theta in (("rope_1e4", 10000.0), ("rope_1e6", 1000000.0)):
        g = rng(16)
        t = {"x": normal(g, (2, 3, 40, 64)), "dY": normal(g, (2, 3, 40, 64))}
        put(name, t, refrun.run_op("rope", t, rope_theta=theta), rope_theta=theta)

    g = rng(17)
    t = {"x": normal(g, (2, 2, 5, 8)), "dY": normal(g, (2, 6, 5, 8))}
    put("repeat_kv", t, refrun.run_op("repeat_kv", t, repeat=3), repeat=3)

    g = rng(18)
    labels = g.integers(0, 50, size=(2, 9)).astype(np.int32)
    labels[0, 3] = -100
    labels[1, 0] = -100
    t = {"logits": normal(g, (2, 9, 50), 2.0), "labels": labels}
    put("lm_ce", t, refrun.run_op("lm_ce", t, ignore_index=-100))
    labels = g.integers(0, 520, size=(2, 9)).astype(np.int32)
    labels[1, 5] = -100
    t = {"hidden": normal(g, (2, 9, 64)), "W": normal(g, (520, 64), 0.2), "labels": labels}
    put("lm_head_ce", t, refrun.run_op("lm_head_ce", t, ignore_index=-100))
    put("streaming_ce", t, refrun.run_op("streaming_ce", t, ignore_index=-100))
    t_all = dict(t)
    t_all["labels"] = np.full((2, 9), -100, dtype=np.int32)
    put("lm_ce_all_ignored", t_all, refrun.run_op("lm_head_ce", t_all, ignore_index=-100))

    g = rng(19)
    t = {"p": normal(g, (37, 5)), "g0": normal(g, (37, 5)), "g1": normal(g, (37, 5), 0.01), "g2": normal(g, (37, 5), 3.0)}
    put("adam_clip", t, refrun.run_op("adam", t, steps=3, lr=1e-3, max_grad_norm=1.0), steps=3, lr=1e-3, max_grad_norm=1.0)
    put("adam_wd", t, refrun.run_op("adam", t, steps=3, lr=2e-4, weight_decay=0.01), steps=3, lr=2e-4, weight_decay=0.01)

    out = Path(__file__).with_name("ops_golden.npz")
    np.savez_compressed(out, **store)
    print(out, out.stat().st_size, "bytes,", len(store), "arrays; driver:", refrun.kind(refrun.driver()))




def make_model_golden():
    """Whole-model LoRA step of the reference on the reduced cases of tests/model_cases.py.
    Inputs are regenerated from seeds (mobilefinetuner_b200.synth), so only outputs are stored."""
    sys.path.insert(0, str(ROOT / "tests"))
    from model_cases import CASES, STEP
    from mobilefinetuner_b200 import synth
    from oracle import model_case
    store = {}
    for name, c in CASES.items():
        spec = c["spec"]
        params = synth.make_params(spec, c["seeds"][0], c["norm_jitter"])
        lora = synth.make_lora(spec, c["seeds"][1])
        ids, labels = synth.make_batch(spec, c["batch"], c["seq"], c["seeds"][2])
        r = model_case.run_reference_step(spec, params, lora, ids, labels, **STEP)
        store[f"{name}/loss"] = r["loss"]
        for i, g in enumerate(r["grads"]):
            if g is not None:
                store[f"{name}/grad/{i}"] = g
        for i, a in enumerate(r["lora_after"]):
            store[f"{name}/after/{i}"] = a
        print(name, "loss", r["loss"], "tensors", len(lora))
    out = Path(__file__).with_name("model_golden.npz")
    np.savez_compressed(out, **store)
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
    make_model_golden()
