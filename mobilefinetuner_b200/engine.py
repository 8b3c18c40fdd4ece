"""LoRA fine-tuning step engine: Python handle over the C ABI of include/mft_step.h.

Mirrors the reference's step driver (AutoModelForCausalLM + AutoTrainer::train_step,
operator/finetune_ops/optim/auto_trainer.cpp:20-46): parameters()/trainable_parameters()
orders and layouts are the reference's, `train_step` is forward -> lm_cross_entropy ->
backward -> clip -> Adam -> zero_grad.  All compute runs in libmft_cuda.so; torch supplies
pinned host buffers, the stream and (for data parallel runs) torch.distributed.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib as L
from .configs import ModelSpec, StepConfig


class LoraStepEngine:
    def __init__(self, spec: ModelSpec, max_batch: int, max_seq: int, device: int = 0):
        if not torch.cuda.is_available():
            raise L.MftError("no CUDA device: the LoRA step engine has no CPU path")
        torch.cuda.set_device(device)
        L.init(device)
        self.spec, self.device = spec, device
        cfg = L.ModelConfig(
            family=spec.family, vocab=spec.vocab, hidden=spec.hidden, inter=spec.inter, layers=spec.layers,
            n_heads=spec.n_heads, n_kv_heads=spec.n_kv_heads, head_dim=spec.head_dim, n_positions=spec.n_positions,
            norm_eps=spec.norm_eps, rope_theta=spec.rope_theta, rope_local_theta=spec.rope_local_theta,
            attn_scale=spec.attn_scale, sliding_window=spec.sliding_window, global_every=spec.global_every,
            lora_rank=spec.lora_rank, lora_alpha=spec.lora_alpha, lora_targets=spec.lora_mask,
            gpt2_detach_attn=1 if spec.gpt2_detach_attn else 0, max_batch=max_batch, max_seq=max_seq)
        self.stream = torch.cuda.current_stream().cuda_stream
        h = C.c_void_p()
        L.call("mft_model_create", C.byref(cfg), self.stream, C.byref(h))
        self._h = h
        self.max_batch, self.max_seq = max_batch, max_seq
        self._pin_ids = torch.empty(max_batch * max_seq, dtype=torch.int32).pin_memory()
        self._pin_labels = torch.empty(max_batch * max_seq, dtype=torch.int32).pin_memory()
        p, g, n = C.c_void_p(), C.c_void_p(), C.c_int64()
        L.call("mft_model_buckets", self._h, C.byref(p), C.byref(g), C.byref(n))
        self.bucket_n = n.value
        self._grad_ptr, self._param_ptr = g.value, p.value

    def close(self):
        if getattr(self, "_h", None):
            L.call("mft_model_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters (reference order and layout)
    def param_shapes(self):
        out = []
        for i in range(L.call("mft_model_param_count", self._h)):
            r, c = C.c_int64(), C.c_int64()
            L.call("mft_model_param_shape", self._h, i, C.byref(r), C.byref(c))
            out.append((r.value, c.value))
        return out

    def lora_shapes(self):
        out = []
        for i in range(L.call("mft_model_lora_count", self._h)):
            r, c = C.c_int64(), C.c_int64()
            L.call("mft_model_lora_shape", self._h, i, C.byref(r), C.byref(c))
            out.append((r.value, c.value))
        return out

    def set_params(self, arrays):
        shapes = self.param_shapes()
        assert len(arrays) == len(shapes), (len(arrays), len(shapes))
        for i, (a, (r, c)) in enumerate(zip(arrays, shapes)):
            if isinstance(a, torch.Tensor):
                assert a.is_cuda and a.dtype == torch.float32 and a.numel() == r * c
                L.call("mft_model_set_param_dev", self._h, i, a.contiguous().data_ptr())
            else:
                a = np.ascontiguousarray(a, dtype=np.float32)
                assert a.size == r * c, (i, a.shape, (r, c))
                L.call("mft_model_set_param_host", self._h, i, a.ctypes.data)
        torch.cuda.synchronize()

    def set_lora(self, arrays):
        shapes = self.lora_shapes()
        assert len(arrays) == len(shapes), (len(arrays), len(shapes))
        for i, (a, (r, c)) in enumerate(zip(arrays, shapes)):
            a = np.ascontiguousarray(a, dtype=np.float32)
            assert a.shape == (r, c), (i, a.shape, (r, c))
            L.call("mft_model_set_lora_host", self._h, i, a.ctypes.data)

    def get_lora(self):
        out = []
        for i, (r, c) in enumerate(self.lora_shapes()):
            a = np.empty((r, c), np.float32)
            L.call("mft_model_get_lora_host", self._h, i, a.ctypes.data)
            out.append(a)
        return out

    def get_lora_grads(self):
        out = []
        for i, (r, c) in enumerate(self.lora_shapes()):
            if not L.call("mft_model_lora_has_grad", self._h, i):
                out.append(None)
                continue
            a = np.empty((r, c), np.float32)
            L.call("mft_model_get_lora_grad_host", self._h, i, a.ctypes.data)
            out.append(a)
        return out

    def grad_bucket(self) -> torch.Tensor:
        """The flat f32 LoRA-gradient bucket as a torch view (what data parallel all-reduces)."""
        return _as_tensor(self._grad_ptr, self.bucket_n, self.device)

    def param_bucket(self) -> torch.Tensor:
        return _as_tensor(self._param_ptr, self.bucket_n, self.device)

    # ---- the step
    def forward_backward(self, ids: np.ndarray, labels: np.ndarray, n_valid_global: int = 0):
        b, s = ids.shape
        n = b * s
        self._pin_ids[:n].copy_(torch.from_numpy(np.ascontiguousarray(ids, np.int32).ravel()))
        self._pin_labels[:n].copy_(torch.from_numpy(np.ascontiguousarray(labels, np.int32).ravel()))
        return self.forward_backward_pinned(b, s, n_valid_global)

    def forward_backward_pinned(self, b: int, s: int, n_valid_global: int = 0):
        """ids / labels were already written to self._pin_ids / self._pin_labels."""
        loss, nv = C.c_float(), C.c_int32()
        L.call("mft_model_forward_backward", self._h, self._pin_ids.data_ptr(), self._pin_labels.data_ptr(), b, s,
               int(n_valid_global), C.byref(loss), C.byref(nv))
        return loss.value, nv.value

    def forward_loss(self, ids: np.ndarray, labels: np.ndarray) -> float:
        b, s = ids.shape
        ids = np.ascontiguousarray(ids, np.int32)
        labels = np.ascontiguousarray(labels, np.int32)
        loss = C.c_float()
        L.call("mft_model_forward_loss", self._h, ids.ctypes.data, labels.ctypes.data, b, s, C.byref(loss))
        return loss.value

    # ---- evaluation drivers
    def perplexity(self, batches):
        """eval_ppl of the reference over an iterable of (ids, labels): returns (mean_nll, ppl, tokens)."""
        acc = L.PplAccum(0.0, 0, 0)
        for ids, labels in batches:
            b, s = ids.shape
            ids = np.ascontiguousarray(ids, np.int32)
            labels = np.ascontiguousarray(labels, np.int32)
            L.call("mft_model_eval_ppl_batch", self._h, C.byref(acc), ids.ctypes.data, labels.ctypes.data, b, s)
        nll, ppl = C.c_float(), C.c_float()
        L.call("mft_ppl_result", C.byref(acc), C.byref(nll), C.byref(ppl))
        return nll.value, ppl.value, acc.sum_tokens

    def score_tokens(self, prompt_ids, candidate_ids) -> np.ndarray:
        """log p(candidate | prompt) at the prompt's last position (MMLU letter scoring)."""
        ids = np.ascontiguousarray(prompt_ids, np.int32).ravel()
        cand = np.ascontiguousarray(candidate_ids, np.int32).ravel()
        out = np.empty(cand.size, np.float32)
        L.call("mft_model_score_tokens", self._h, ids.ctypes.data, ids.size, cand.ctypes.data, cand.size, out.ctypes.data)
        return out

    def merge_to_base(self):
        """Fold scale * A B into the device weights (LoRALinear::merge_to_base, nn/lora_linear.cpp:470-483); forward and
        evaluation calls then skip the adapter products, training calls raise until unmerge_from_base()."""
        L.call("mft_model_merge_lora", self._h)

    def unmerge_from_base(self):
        """Restore the weights saved by merge_to_base() byte for byte (nn/lora_linear.cpp:485-508)."""
        L.call("mft_model_unmerge_lora", self._h)

    @property
    def is_merged(self) -> bool:
        return bool(L.load().mft_model_is_merged(self._h))

    def optimizer_step(self, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, max_grad_norm=0.0, clip_eps=0.0):
        L.call("mft_model_optimizer_step", self._h, float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
               float(max_grad_norm), float(clip_eps))

    def zero_grad(self):
        L.call("mft_model_zero_grad", self._h)

    def train_step(self, ids, labels, cfg: StepConfig, world=None):
        """forward + loss + backward (+ all-reduce of the LoRA gradients) + clip + Adam + zero_grad."""
        n_global = 0
        if world is not None and world.size > 1:
            n_global = world.global_valid_count(labels)
        loss, _ = self.forward_backward(ids, labels, n_global)
        if world is not None and world.size > 1:
            world.all_reduce_sum(self.grad_bucket())
        self.optimizer_step(cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.max_grad_norm, 0.0)
        return loss

    def final_hidden(self, n_tokens: int) -> np.ndarray:
        out = np.empty((n_tokens, self.spec.hidden), np.float32)
        L.call("mft_model_get_final_hidden_host", self._h, out.ctypes.data, out.size)
        return out

    def activation_bytes(self) -> int:
        return L.call("mft_model_activation_bytes", self._h)


class LoraTrainer:
    """The step driver of the reference's trainers (GemmaLoRATrainer / LoRATrainer ::train_step) over a
    LoraStepEngine: micro-batches accumulate gradients on the device with the loss scaled by 1/grad_accum_steps;
    every grad_accum_steps-th call clips, sets the scheduled learning rate, runs Adam and clears the gradients."""

    def __init__(self, engine: LoraStepEngine, *, learning_rate=2e-4, weight_decay=0.0, adam_beta1=0.9, adam_beta2=0.999,
                 adam_eps=1e-8, max_grad_norm=1.0, lr_scheduler="linear", warmup_ratio=0.03, grad_accum_steps=1,
                 num_sequences=None, micro_batch_size=1, num_epochs=3, total_updates=None):
        if total_updates is None:
            micro_per_epoch = (int(num_sequences) + micro_batch_size - 1) // micro_batch_size
            total_updates = max(1, (micro_per_epoch * num_epochs + grad_accum_steps - 1) // grad_accum_steps)
        self.engine = engine
        self.cfg = L.TrainerConfig(learning_rate, weight_decay, adam_beta1, adam_beta2, adam_eps, max_grad_norm, warmup_ratio,
                                   L.LR_SCHEDULERS[lr_scheduler], grad_accum_steps, total_updates)
        h = C.c_void_p()
        L.call("mft_trainer_create", engine._h, C.byref(self.cfg), C.byref(h))
        self._h = h

    def lr(self, step: int) -> float:
        return L.call("mft_trainer_lr", C.byref(self.cfg), int(step))

    @property
    def global_step(self) -> int:
        return L.call("mft_trainer_global_step", self._h)

    def train_step(self, ids: np.ndarray, labels: np.ndarray, n_valid_global: int = 0):
        """Returns the mean loss of the accumulation window when this call closed it, else -1.0 (as the reference)."""
        b, s = ids.shape
        ids = np.ascontiguousarray(ids, np.int32)
        labels = np.ascontiguousarray(labels, np.int32)
        stepped, loss, lr = C.c_int32(), C.c_float(), C.c_float()
        L.call("mft_trainer_train_step", self._h, ids.ctypes.data, labels.ctypes.data, b, s, int(n_valid_global),
               C.byref(stepped), C.byref(loss), C.byref(lr))
        self.last_lr = lr.value if stepped.value else None
        return loss.value if stepped.value else -1.0

    def close(self):
        if self._h:
            L.call("mft_trainer_destroy", self._h)
            self._h = None


class BatchPipeline:
    """Double-buffered input for a LoraStepEngine: while step k computes, batch k+1 is copied from page-locked host
    buffers to the device on a copy stream, and the loss of step k is read back one step later, so the GPU never
    waits for the host between steps.  The host buffers play the role of the reusable Batch buffers of
    WikiText2Dataset::get_batch."""

    def __init__(self, engine: LoraStepEngine, batch: int, seq: int):
        self.engine, self.batch, self.seq = engine, batch, seq
        n = batch * seq
        self.ids = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.labels = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.loss = torch.zeros(2, dtype=torch.float32).pin_memory()
        self.n_valid = torch.zeros(2, dtype=torch.int32).pin_memory()

    def _stage(self, slot, ids, labels):
        self.ids[slot].copy_(torch.from_numpy(np.ascontiguousarray(ids, np.int32).ravel()))
        self.labels[slot].copy_(torch.from_numpy(np.ascontiguousarray(labels, np.int32).ravel()))
        L.call("mft_model_stage_batch", self.engine._h, slot, self.ids[slot].data_ptr(), self.labels[slot].data_ptr(),
               self.batch, self.seq)

    def run(self, batches, after_backward=None, n_valid_global=0):
        """Runs forward + backward on every (ids, labels) of `batches`; `after_backward(k)` (e.g. the optimizer step)
        is queued right after step k.  Yields (k, loss, n_valid) for every step, one step late."""
        h = self.engine._h
        it = iter(batches)
        try:
            first = next(it)
        except StopIteration:
            return
        self._stage(0, *first)
        done, pending, used = None, None, [True, False]
        k, slot = 0, 0
        while True:
            nxt = next(it, None)
            L.call("mft_model_step_staged", h, slot, self.batch, self.seq, int(n_valid_global),
                   self.loss[slot:].data_ptr(), self.n_valid[slot:].data_ptr())
            ev = torch.cuda.Event()
            ev.record()
            if after_backward is not None:
                after_backward(k)
            if nxt is not None:
                other = slot ^ 1
                if used[other]:
                    L.call("mft_model_stage_wait", h, other)      # its previous copy has left the host buffers
                self._stage(other, *nxt)
                used[other] = True
            if pending is not None:                               # results of the step before: already complete or nearly
                pk, pslot, pev = pending
                pev.synchronize()
                yield pk, float(self.loss[pslot]), int(self.n_valid[pslot])
            pending = (k, slot, ev)
            if nxt is None:
                break
            k, slot = k + 1, slot ^ 1
        pk, pslot, pev = pending
        pev.synchronize()
        L.call("mft_model_sync", h)
        yield pk, float(self.loss[pslot]), int(self.n_valid[pslot])


def _as_tensor(ptr: int, n: int, device: int) -> torch.Tensor:
    """Wrap device memory owned by the engine as a 1-D float32 torch tensor (no copy)."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}
    return torch.as_tensor(h, device=f"cuda:{device}")
