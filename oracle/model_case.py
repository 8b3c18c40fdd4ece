"""Test infrastructure: drives the compiled reference (oracle/_ref/ref_driver_*) through one
whole-model LoRA step on given parameters and a batch, the way
graph/test_auto_model.cpp:63-91 does (config.json -> from_pretrained(load_weights=false) ->
overwrite parameters() -> init_lora -> overwrite trainable_parameters() -> forward ->
lm_cross_entropy -> backward -> clip -> Adam).  Never imported by the product."""
from __future__ import annotations

from pathlib import Path

import numpy as np

from . import refrun


def run_reference_step(spec, params, lora, ids, labels, *, lr=2e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                       max_grad_norm=0.0, steps=1, update=True, dump_logits=False, threads=None, keep: Path | None = None,
                       prefer_blas=True, timeout=7200):
    """Returns {"loss": [steps], "grads": [...or None], "lora_after": [...], "timing": str, "driver": "blas"|"noblas"}."""
    tensors = {"input_ids": np.ascontiguousarray(ids, np.int32), "labels": np.ascontiguousarray(labels, np.int32),
               "attention_mask": np.ones(ids.shape, np.float32)}
    for i, a in enumerate(params):
        tensors[f"params/{i:04d}"] = np.ascontiguousarray(a, np.float32)
    for i, a in enumerate(lora):
        tensors[f"lora/{i:04d}"] = np.ascontiguousarray(a, np.float32)
    p = {"lora_rank": spec.lora_rank, "lora_alpha": spec.lora_alpha, "lora_targets": ",".join(spec.lora_targets),
         "gpt2_split_qkv": 0, "lr": lr, "beta1": beta1, "beta2": beta2, "eps": eps, "weight_decay": weight_decay,
         "max_grad_norm": max_grad_norm, "steps": steps, "update": 1 if update else 0, "dump_logits": 1 if dump_logits else 0}
    out = refrun.run("model", p, tensors, extra_files={"config.json": spec.config_json()}, threads=threads, keep=keep,
                     prefer_blas=prefer_blas, timeout=timeout)
    n = len(lora)
    res = {"loss": out["loss"], "grads": [out.get(f"grad_{i:04d}") for i in range(n)],
           "lora_after": [out[f"lora_after_{i:04d}"] for i in range(n)], "timing": out.get("_timing", ""),
           "driver": out["_driver"]}
    if dump_logits:
        res["logits"] = out["logits"]
    return res
