"""Architectures of the three model families the LoRA step supports, and the
benchmark configurations (sizes, LoRA targets, batch shapes).

Field names follow the reference's config parsers
(operator/finetune_ops/graph/gpt2_model.cpp:56-75, qwen_model.cpp:40-78,
gemma_model.cpp:138-171) so a `config.json` written from a ModelSpec is what
AutoModelForCausalLM::from_pretrained reads.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, replace

GPT2, QWEN, GEMMA = 0, 1, 2
LORA_BITS = {"q": 1, "k": 2, "v": 4, "o": 8, "gate": 16, "up": 32, "down": 64}
# reference module names -> bit
_GPT2_NAMES = {"c_attn": "q", "c_proj": "o", "c_fc": "gate", "mlp_c_proj": "down"}
_HF_NAMES = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "o_proj": "o", "gate_proj": "gate", "up_proj": "up", "down_proj": "down"}


@dataclass(frozen=True)
class ModelSpec:
    family: int
    vocab: int
    hidden: int
    inter: int
    layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    n_positions: int = 0
    norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_local_theta: float = 10000.0
    query_pre_attn_scalar: float = 0.0      # Gemma; 0 -> head_dim
    sliding_window: int = 0
    global_every: int = 0                   # Gemma: layer i global iff (i+1) % global_every == 0
    lora_rank: int = 8
    lora_alpha: float = 16.0
    lora_targets: tuple = ()
    gpt2_detach_attn: bool = True
    weights_bf16: bool = True               # frozen weights are bf16-rounded values
    name: str = ""

    @property
    def attn_scale(self) -> float:
        if self.family == GEMMA:
            return float((self.query_pre_attn_scalar or self.head_dim) ** -0.5)
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def lora_mask(self) -> int:
        names = _GPT2_NAMES if self.family == GPT2 else _HF_NAMES
        m = 0
        for t in self.lora_targets:
            m |= LORA_BITS[names[t]]
        return m

    def layer_is_sliding(self, i: int) -> bool:
        return self.family == GEMMA and not (self.global_every > 0 and (i + 1) % self.global_every == 0)

    def config_json(self) -> str:
        """The config.json the reference's from_pretrained parses for this architecture."""
        if self.family == GPT2:
            d = {"model_type": "gpt2", "vocab_size": self.vocab, "n_positions": self.n_positions, "n_embd": self.hidden,
                 "n_layer": self.layers, "n_head": self.n_heads, "layer_norm_epsilon": 1e-5}
        elif self.family == QWEN:
            d = {"model_type": "qwen2", "vocab_size": self.vocab, "hidden_size": self.hidden, "intermediate_size": self.inter,
                 "num_hidden_layers": self.layers, "num_attention_heads": self.n_heads, "num_key_value_heads": self.n_kv_heads,
                 "max_position_embeddings": 32768, "rms_norm_eps": self.norm_eps, "rope_theta": float(self.rope_theta)}
        else:
            d = {"model_type": "gemma3_text", "vocab_size": self.vocab, "hidden_size": self.hidden, "intermediate_size": self.inter,
                 "num_hidden_layers": self.layers, "num_attention_heads": self.n_heads, "num_key_value_heads": self.n_kv_heads,
                 "head_dim": self.head_dim, "sliding_window": self.sliding_window, "rms_norm_eps": self.norm_eps,
                 "query_pre_attn_scalar": float(self.query_pre_attn_scalar or self.head_dim), "rope_theta": float(self.rope_theta),
                 "rope_local_base_freq": float(self.rope_local_theta),
                 "layer_types": ["sliding_attention" if self.layer_is_sliding(i) else "full_attention" for i in range(self.layers)]}
        return json.dumps(d)

    # ---- shapes in the reference's parameters() / get_lora_parameters() order
    def param_shapes(self) -> list[tuple[str, tuple]]:
        H, I, V = self.hidden, self.inter, self.vocab
        QD, KD = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = []
        if self.family == GPT2:
            out += [("wte", (V, H)), ("wpe", (self.n_positions, H))]
            for _ in range(self.layers):
                out += [("ln", (H,)), ("ln_b", (H,)), ("linear", (H, 3 * H)), ("bias", (3 * H,)), ("linear", (H, H)), ("bias", (H,)),
                        ("ln", (H,)), ("ln_b", (H,)), ("linear", (H, I)), ("bias", (I,)), ("linear", (I, H)), ("bias", (H,))]
            out += [("ln", (H,)), ("ln_b", (H,))]
        elif self.family == QWEN:
            out += [("embed", (V, H)), ("norm", (H,))]
            for _ in range(self.layers):
                out += [("norm", (H,)), ("norm", (H,)), ("linear", (H, QD)), ("bias", (QD,)), ("linear", (H, KD)), ("bias", (KD,)),
                        ("linear", (H, KD)), ("bias", (KD,)), ("linear", (QD, H)), ("linear", (H, I)), ("linear", (H, I)), ("linear", (I, H))]
        else:
            out += [("embed", (V, H)), ("norm", (H,)), ("lm_head", (H, V))]
            for _ in range(self.layers):
                out += [("norm", (H,))] * 4 + [("linear", (H, QD)), ("linear", (H, KD)), ("linear", (H, KD)), ("linear", (QD, H)),
                                                ("norm", (self.head_dim,)), ("norm", (self.head_dim,)),
                                                ("linear", (H, I)), ("linear", (H, I)), ("linear", (I, H))]
        return out

    def lora_shapes(self) -> list[tuple[str, tuple]]:
        H, I, r = self.hidden, self.inter, self.lora_rank
        QD, KD = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        if self.family == GPT2:
            dims = {"c_attn": (H, 3 * H), "c_proj": (H, H), "c_fc": (H, I), "mlp_c_proj": (I, H)}
            order = ["c_attn", "c_proj", "c_fc", "mlp_c_proj"]
        elif self.family == QWEN:
            dims = {"q_proj": (H, QD), "v_proj": (H, KD), "k_proj": (H, KD), "o_proj": (QD, H)}
            order = ["q_proj", "v_proj", "k_proj", "o_proj"]
        else:
            dims = {"q_proj": (H, QD), "k_proj": (H, KD), "v_proj": (H, KD), "o_proj": (QD, H),
                    "gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
            order = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
        out = []
        for _ in range(self.layers):
            for name in order:
                if name not in self.lora_targets:
                    continue
                i, o = dims[name]
                if self.family == GEMMA:
                    out += [(name + ".A", (r, i)), (name + ".B", (o, r))]
                else:
                    out += [(name + ".A", (i, r)), (name + ".B", (r, o))]
        return out

    def step_flops(self, batch: int, seq: int) -> float:
        """Algorithmic FLOPs of one step (2 per MAC; no recomputation, masked attention pairs not counted)."""
        T = batch * seq
        H, I = self.hidden, self.inter
        QD, KD = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        if self.family == GPT2:
            lin = {"c_attn": (H, 3 * H), "c_proj": (H, H), "c_fc": (H, I), "mlp_c_proj": (I, H)}
        else:
            lin = {"q_proj": (H, QD), "k_proj": (H, KD), "v_proj": (H, KD), "o_proj": (QD, H), "gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
        p_lin = sum(a * b for a, b in lin.values())
        p_lora = sum(self.lora_rank * (a + b) for n, (a, b) in lin.items() if n in self.lora_targets)
        f = T * self.layers * (4.0 * p_lin + 6.0 * p_lora)
        for i in range(self.layers):
            if self.layer_is_sliding(i) and self.sliding_window > 0:
                pairs = sum(min(j + 1, self.sliding_window) for j in range(seq))
            else:
                pairs = seq * (seq + 1) // 2
            f += 12.0 * self.head_dim * self.n_heads * batch * pairs
        f += 4.0 * T * H * self.vocab
        return f


GPT2_SMALL = ModelSpec(family=GPT2, vocab=50257, hidden=768, inter=3072, layers=12, n_heads=12, n_kv_heads=12, head_dim=64,
                       n_positions=1024, norm_eps=1e-5, lora_rank=8, lora_alpha=16.0, lora_targets=("c_attn", "c_proj"),
                       weights_bf16=False, name="gpt2-small")
QWEN25_05B = ModelSpec(family=QWEN, vocab=151936, hidden=896, inter=4864, layers=24, n_heads=14, n_kv_heads=2, head_dim=64,
                       norm_eps=1e-6, rope_theta=1e6, lora_rank=16, lora_alpha=32.0, lora_targets=("q_proj", "k_proj", "v_proj", "o_proj"),
                       name="qwen2.5-0.5b")
_GEMMA_ALL = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
GEMMA3_270M = ModelSpec(family=GEMMA, vocab=262144, hidden=640, inter=2048, layers=18, n_heads=4, n_kv_heads=1, head_dim=256,
                        norm_eps=1e-6, rope_theta=1e6, rope_local_theta=1e4, query_pre_attn_scalar=256.0, sliding_window=512,
                        global_every=6, lora_rank=8, lora_alpha=32.0, lora_targets=_GEMMA_ALL, name="gemma-3-270m")
GEMMA3_1B = ModelSpec(family=GEMMA, vocab=262144, hidden=1152, inter=6912, layers=26, n_heads=4, n_kv_heads=1, head_dim=256,
                      norm_eps=1e-6, rope_theta=1e6, rope_local_theta=1e4, query_pre_attn_scalar=256.0, sliding_window=512,
                      global_every=6, lora_rank=16, lora_alpha=32.0, lora_targets=_GEMMA_ALL, name="gemma-3-1b")


@dataclass(frozen=True)
class StepConfig:
    name: str
    spec: ModelSpec
    batch: int
    seq: int
    lr: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    seed: int = 0


CONFIGS = {
    "gpt2_small": StepConfig("gpt2_small", GPT2_SMALL, 4, 128, seed=1),
    "qwen25_05b": StepConfig("qwen25_05b", QWEN25_05B, 8, 512, seed=3),
    "gemma3_270m": StepConfig("gemma3_270m", GEMMA3_270M, 16, 1024, seed=4),
    "gemma3_1b": StepConfig("gemma3_1b", GEMMA3_1B, 8, 2048, seed=5),
}


def reduced(spec: ModelSpec, **changes) -> ModelSpec:
    """A smaller model of the same architecture (parity cases the CPU reference can hold)."""
    return replace(spec, **changes)
