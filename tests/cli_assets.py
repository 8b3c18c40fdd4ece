"""Synthetic assets for running the reference's command-line programs end to end: a small GPT-2 checkpoint directory
(config.json, model.safetensors with HuggingFace keys, a byte-level vocab.json with no merges), a WikiText-style text
file and a LoRA adapter file in the layout of the reference's LoraSaver.  Everything is seeded; nothing is downloaded."""
import json
from pathlib import Path

import numpy as np

from test_safetensors_cpu import write_container


def bytes_to_unicode():
    """The byte -> printable character table of GPT-2's byte-level BPE."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, (chr(c) for c in cs)))


GPT2_TINY = dict(n_layer=2, n_embd=64, n_head=4, n_positions=128, vocab_size=50257)


def write_gpt2_checkpoint(root: Path, seed: int = 7, scale: float = 0.08) -> dict:
    """Returns the tensors written (HF key -> f32 array, Linear weights [in, out] as GPT-2 stores them)."""
    c = GPT2_TINY
    root.mkdir(parents=True, exist_ok=True)
    (root / "config.json").write_text(json.dumps({"model_type": "gpt2", "n_layer": c["n_layer"], "n_embd": c["n_embd"], "n_head": c["n_head"],
                                                  "n_positions": c["n_positions"], "n_ctx": c["n_positions"], "vocab_size": c["vocab_size"],
                                                  "layer_norm_epsilon": 1e-5}))
    vocab = {ch: i for i, (_, ch) in enumerate(sorted(bytes_to_unicode().items()))}     # token id = byte value
    vocab["<|endoftext|>"] = 50256
    (root / "vocab.json").write_text(json.dumps(vocab))
    (root / "merges.txt").write_text("#version: 0.2\n")
    rng = np.random.default_rng(seed)
    E, V, P = c["n_embd"], c["vocab_size"], c["n_positions"]
    t = {"wte.weight": rng.normal(0, scale, (V, E)), "wpe.weight": rng.normal(0, scale, (P, E)),
         "ln_f.weight": 1 + rng.normal(0, 0.05, E), "ln_f.bias": rng.normal(0, 0.02, E)}
    for i in range(c["n_layer"]):
        h = f"h.{i}."
        t[h + "ln_1.weight"] = 1 + rng.normal(0, 0.05, E); t[h + "ln_1.bias"] = rng.normal(0, 0.02, E)
        t[h + "ln_2.weight"] = 1 + rng.normal(0, 0.05, E); t[h + "ln_2.bias"] = rng.normal(0, 0.02, E)
        t[h + "attn.c_attn.weight"] = rng.normal(0, scale, (E, 3 * E)); t[h + "attn.c_attn.bias"] = rng.normal(0, 0.02, 3 * E)
        t[h + "attn.c_proj.weight"] = rng.normal(0, scale, (E, E)); t[h + "attn.c_proj.bias"] = rng.normal(0, 0.02, E)
        t[h + "mlp.c_fc.weight"] = rng.normal(0, scale, (E, 4 * E)); t[h + "mlp.c_fc.bias"] = rng.normal(0, 0.02, 4 * E)
        t[h + "mlp.c_proj.weight"] = rng.normal(0, scale, (4 * E, E)); t[h + "mlp.c_proj.bias"] = rng.normal(0, 0.02, E)
    t = {k: np.ascontiguousarray(v, np.float32) for k, v in t.items()}
    write_container(root / "model.safetensors", {k: ("F32", v) for k, v in t.items()}, {"format": "pt"})
    return t


def write_text_corpus(root: Path, seed: int = 11, n_lines: int = 60):
    """wiki.{train,valid,test}.raw: lines of seeded pseudo-words (ASCII), a heading line now and then."""
    rng = np.random.default_rng(seed)
    words = ["".join(chr(97 + int(x)) for x in rng.integers(0, 26, int(rng.integers(2, 9)))) for _ in range(200)]
    root.mkdir(parents=True, exist_ok=True)
    for split in ("train", "valid", "test"):
        lines = []
        for i in range(n_lines):
            if i % 15 == 0:
                lines.append(f" = {words[int(rng.integers(0, 200))].capitalize()} = ")
            lines.append(" " + " ".join(words[int(x)] for x in rng.integers(0, 200, int(rng.integers(8, 30)))) + " . ")
        (root / f"wiki.{split}.raw").write_text("\n".join(lines) + "\n")


def write_gpt2_adapter(path: Path, seed: int = 13, rank: int = 4, alpha: float = 8.0, scale: float = 0.5):
    """Adapter on attn.proj, mlp.fc_in and mlp.fc_out of every layer: A [in, r], B [r, out], both non-zero."""
    c = GPT2_TINY
    E = c["n_embd"]
    rng = np.random.default_rng(seed)
    dims = {"attn.proj": (E, E), "mlp.fc_in": (E, 4 * E), "mlp.fc_out": (4 * E, E)}
    t = {}
    for i in range(c["n_layer"]):
        for name, (din, dout) in dims.items():
            t[f"layer.{i}.{name}.lora_A"] = ("F32", np.ascontiguousarray(rng.normal(0, scale, (din, rank)), np.float32))
            t[f"layer.{i}.{name}.lora_B"] = ("F32", np.ascontiguousarray(rng.normal(0, scale, (rank, dout)), np.float32))
    write_container(path, t, {"rank": str(rank), "alpha": str(alpha), "dropout": "0", "split_qkv": "true", "targets": "AttnProj,MlpFcIn,MlpFcOut"})


def read_container(path: Path) -> dict:
    """F32 tensors of a safetensors file as name -> ndarray (metadata dropped)."""
    import struct
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        assert e["dtype"] == "F32", (name, e["dtype"])
        a, b = e["data_offsets"]
        out[name] = np.frombuffer(raw[8 + n + a:8 + n + b], np.float32).reshape(e["shape"]).copy()
    return out


QWEN_TINY = dict(num_hidden_layers=2, hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, vocab_size=151936)


def write_qwen_checkpoint(root: Path, seed: int = 17, scale: float = 0.15) -> dict:
    """A Qwen2-style model directory: config.json, byte-level vocab.json / merges.txt, tokenizer.json with the
    <|endoftext|> added token (id 151643, as the reference's tokenizer assumes), model.safetensors with HuggingFace keys
    (Linear weights [out, in], q / k / v biases).  Returns the tensors written."""
    c = QWEN_TINY
    root.mkdir(parents=True, exist_ok=True)
    H, I, V, nh, nkv = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["num_attention_heads"], c["num_key_value_heads"]
    hd = H // nh
    (root / "config.json").write_text(json.dumps({"model_type": "qwen2", "hidden_size": H, "intermediate_size": I, "num_hidden_layers": c["num_hidden_layers"],
                                                  "num_attention_heads": nh, "num_key_value_heads": nkv, "vocab_size": V, "max_position_embeddings": 512,
                                                  "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "hidden_act": "silu", "tie_word_embeddings": True,
                                                  "eos_token_id": 151643, "bos_token_id": 151643}))
    vocab = {ch: i for i, (_, ch) in enumerate(sorted(bytes_to_unicode().items()))}
    (root / "vocab.json").write_text(json.dumps(vocab))
    (root / "merges.txt").write_text("#version: 0.2\n")
    (root / "tokenizer.json").write_text(json.dumps({"added_tokens": [{"id": 151643, "content": "<|endoftext|>", "single_word": False, "lstrip": False,
                                                                       "rstrip": False, "normalized": False, "special": True}],
                                                     "model": {"type": "BPE"}}))
    rng = np.random.default_rng(seed)
    t = {"model.embed_tokens.weight": rng.normal(0, scale, (V, H)), "model.norm.weight": 1 + rng.normal(0, 0.05, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = 1 + rng.normal(0, 0.05, H)
        t[p + "post_attention_layernorm.weight"] = 1 + rng.normal(0, 0.05, H)
        for name, out in (("q_proj", nh * hd), ("k_proj", nkv * hd), ("v_proj", nkv * hd)):
            t[p + f"self_attn.{name}.weight"] = rng.normal(0, scale, (out, H))
            t[p + f"self_attn.{name}.bias"] = rng.normal(0, 0.02, out)
        t[p + "self_attn.o_proj.weight"] = rng.normal(0, scale, (H, nh * hd))
        t[p + "mlp.gate_proj.weight"] = rng.normal(0, scale, (I, H))
        t[p + "mlp.up_proj.weight"] = rng.normal(0, scale, (I, H))
        t[p + "mlp.down_proj.weight"] = rng.normal(0, scale, (H, I))
    t = {k: np.ascontiguousarray(v, np.float32) for k, v in t.items()}
    write_container(root / "model.safetensors", {k: ("F32", v) for k, v in t.items()}, {"format": "pt"})
    return t


def read_lora_weights_bin(path: Path) -> list:
    """The adapter dump of the reference's Qwen programs: int32 count, then per tensor int32 ndim, int64 dims, f32 data."""
    import struct
    raw = Path(path).read_bytes()
    (n,), off, out = struct.unpack_from("<i", raw, 0), 4, []
    for _ in range(n):
        (nd,) = struct.unpack_from("<i", raw, off); off += 4
        dims = struct.unpack_from(f"<{nd}q", raw, off); off += 8 * nd
        cnt = int(np.prod(dims))
        out.append(np.frombuffer(raw, np.float32, cnt, off).reshape(dims).copy()); off += 4 * cnt
    assert off == len(raw)
    return out


GEMMA_TINY = dict(num_hidden_layers=2, hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=1, head_dim=16,
                  vocab_size=512, sliding_window=32)


def write_gemma_checkpoint(root: Path, seed: int = 19, scale: float = 0.15) -> dict:
    """A Gemma-3-text-style model directory (config.json with one sliding and one full-attention layer, model.safetensors with
    HuggingFace keys: [out, in] linears, q / k norms, the four norms per layer) and a pretokenized corpus next to it
    (tokens.bin int32 + meta.json with the split ranges), which the reference's Gemma program reads instead of
    tokenizing text.  Returns the tensors written."""
    c = GEMMA_TINY
    root.mkdir(parents=True, exist_ok=True)
    H, I, V, nh, nkv, hd = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    (root / "config.json").write_text(json.dumps({
        "model_type": "gemma3_text", "vocab_size": V, "hidden_size": H, "intermediate_size": I, "num_hidden_layers": c["num_hidden_layers"],
        "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "max_position_embeddings": 512, "sliding_window": c["sliding_window"],
        "rms_norm_eps": 1e-6, "query_pre_attn_scalar": float(hd), "rope_theta": 1000000.0, "rope_local_base_freq": 10000.0,
        "hidden_activation": "gelu_pytorch_tanh", "attention_bias": False, "layer_types": ["sliding_attention", "full_attention"],
        "tie_word_embeddings": True}))
    rng = np.random.default_rng(seed)
    t = {"model.embed_tokens.weight": rng.normal(0, scale, (V, H)), "model.norm.weight": rng.normal(0, 0.05, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            t[p + n + ".weight"] = rng.normal(0, 0.05, H)                      # (1 + w) norms: stored around zero
        t[p + "self_attn.q_proj.weight"] = rng.normal(0, scale, (nh * hd, H))
        t[p + "self_attn.k_proj.weight"] = rng.normal(0, scale, (nkv * hd, H))
        t[p + "self_attn.v_proj.weight"] = rng.normal(0, scale, (nkv * hd, H))
        t[p + "self_attn.o_proj.weight"] = rng.normal(0, scale, (H, nh * hd))
        t[p + "self_attn.q_norm.weight"] = rng.normal(0, 0.05, hd)
        t[p + "self_attn.k_norm.weight"] = rng.normal(0, 0.05, hd)
        t[p + "mlp.gate_proj.weight"] = rng.normal(0, scale, (I, H))
        t[p + "mlp.up_proj.weight"] = rng.normal(0, scale, (I, H))
        t[p + "mlp.down_proj.weight"] = rng.normal(0, scale, (H, I))
    t = {k: np.ascontiguousarray(v, np.float32) for k, v in t.items()}
    write_container(root / "model.safetensors", {k: ("F32", v) for k, v in t.items()}, {"format": "pt"})
    return t


def write_pretokenized_corpus(root: Path, vocab: int, seed: int = 23, n_train: int = 6000, n_valid: int = 1500):
    """tokens.bin (int32, train then valid) + meta.json: Zipf-distributed ids in [4, vocab), an end-of-text id 1 now and then."""
    root.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    ids = (4 + (rng.zipf(1.3, n_train + n_valid) - 1) % (vocab - 4)).astype(np.int32)
    ids[rng.random(ids.size) < 0.02] = 1
    ids.tofile(root / "tokens.bin")
    (root / "meta.json").write_text(json.dumps({"total_tokens": int(ids.size), "eos_token_id": 1, "pad_token_id": 0, "bos_token_id": 2, "unk_token_id": 3,
                                                "vocab_size": vocab, "insert_eos_between_lines": True,
                                                "train": {"offset": 0, "length": n_train}, "valid": {"offset": n_train, "length": n_valid}}))
