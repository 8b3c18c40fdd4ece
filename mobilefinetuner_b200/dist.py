"""Data-parallel plumbing for the LoRA step: one process per GPU, the batch sharded by sample,
and exactly one exchange per step - the sum of the flat LoRA-gradient bucket (plus one scalar:
the global count of scored tokens, so every rank scales its loss gradient by 1/n_global and the
summed bucket IS the global-batch mean gradient).  torch.distributed (NCCL on GPUs, gloo in CPU
tests) carries the collective; nothing else crosses ranks."""
from __future__ import annotations

import datetime
import os

import numpy as np
import torch
import torch.distributed as dist


class World:
    def __init__(self, backend: str | None = None):
        self.size = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if self.size > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            kw = {}
            if self.backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                kw["device_id"] = torch.device("cuda", self.local_rank)
            # a short timeout: a rank that never joins a collective ends the job with an error instead of a long hang
            timeout = datetime.timedelta(seconds=int(os.environ.get("MFT_DIST_TIMEOUT_S", "120")))
            dist.init_process_group(self.backend, rank=self.rank, world_size=self.size, timeout=timeout, **kw)

    @property
    def device(self):
        return torch.device("cuda", self.local_rank) if self.backend == "nccl" else torch.device("cpu")

    def shard(self, n_samples: int) -> slice:
        """Contiguous slice of a global batch owned by this rank (n_samples divisible by size)."""
        if n_samples % self.size:
            raise ValueError("global batch must be divisible by the world size")
        per = n_samples // self.size
        return slice(self.rank * per, (self.rank + 1) * per)

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    def all_reduce_max(self, value: float) -> float:
        if self.size == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def global_valid_count(self, labels: np.ndarray, ignore_index: int = -100) -> int:
        """Scored tokens over all ranks: labels[:, 1:] != ignore_index (the loss shifts internally)."""
        local = int((np.asarray(labels)[:, 1:] != ignore_index).sum())
        if self.size == 1:
            return local
        t = torch.tensor([local], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return int(t.item())

    def barrier(self):
        if self.size > 1:
            dist.barrier()

    def close(self):
        if self.size > 1 and dist.is_initialized():
            dist.destroy_process_group()
