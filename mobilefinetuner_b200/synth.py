"""Seeded synthetic inputs for the LoRA step: token ids with a Zipf(1.1) rank
distribution and random weights of the right shapes.  They stand in for the
WikiText-2 / MMLU batches and the pretrained checkpoints the reference's CLIs
consume (neither is available offline).

Host generation (numpy PCG64) gives bit-identical tensors to every consumer
(the CUDA engine and the CPU reference); device generation (torch) is for
full-size throughput runs where only shapes and value distributions matter.
"""
from __future__ import annotations

import numpy as np

from .configs import GEMMA, GPT2, QWEN, ModelSpec

f32 = np.float32


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16, returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


def zipf_ids(g: np.random.Generator, shape, vocab: int, s: float = 1.1) -> np.ndarray:
    """ids = rank - 1 with p(rank) ~ rank^-s over 1..vocab (inverse-CDF sampling)."""
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    u = g.random(int(np.prod(shape)))
    return np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.int32).reshape(shape)


def make_params(spec: ModelSpec, seed: int, norm_jitter: float = 0.0) -> list[np.ndarray]:
    """Frozen parameters in the reference's parameters() order, fp32 (bf16-rounded values when spec.weights_bf16)."""
    g = rng(seed)
    out = []
    embed = None
    for kind, shape in spec.param_shapes():
        if kind in ("wte", "wpe", "embed", "linear", "bias"):
            a = g.standard_normal(shape, dtype=f32) * f32(0.02)
            if spec.weights_bf16 and kind != "bias":
                a = bf16_round(a)
            if kind in ("wte", "embed"):
                embed = a
        elif kind == "lm_head":
            a = np.ascontiguousarray(embed.T)          # Gemma keeps a transposed copy of the tied table
        elif kind in ("ln",):
            a = np.ones(shape, f32) + (g.standard_normal(shape) * norm_jitter).astype(f32)
        elif kind == "ln_b":
            a = (g.standard_normal(shape) * norm_jitter).astype(f32)
        elif kind == "norm":
            base = 0.0 if spec.family == GEMMA else 1.0
            a = np.full(shape, base, f32) + (g.standard_normal(shape) * norm_jitter).astype(f32)
        else:
            raise ValueError(kind)
        out.append(a)
    return out


def make_lora(spec: ModelSpec, seed: int) -> list[np.ndarray]:
    """LoRA tensors in get_lora_parameters() order.  A: uniform (Kaiming-style bound for GPT-2,
    1/sqrt(in) otherwise); B: N(0, 0.02) instead of the reference's zeros so that dA is non-zero."""
    g = rng(seed)
    out = []
    r = spec.lora_rank
    for name, shape in spec.lora_shapes():
        if name.endswith(".A"):
            fan_in = shape[1] if spec.family == GEMMA else shape[0]
            bound = np.sqrt(6.0 / (fan_in + r)) if spec.family == GPT2 else 1.0 / np.sqrt(fan_in)
            out.append(g.uniform(-bound, bound, shape).astype(f32))
        else:
            out.append((g.standard_normal(shape) * 0.02).astype(f32))
    return out


def make_batch(spec: ModelSpec, batch: int, seq: int, seed: int):
    g = rng(seed)
    ids = zipf_ids(g, (batch, seq), spec.vocab)
    return ids, ids.copy()      # labels = input_ids; the loss shifts internally
