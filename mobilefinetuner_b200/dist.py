"""Data-parallel plumbing for the LoRA step: one process per GPU, the batch sharded by sample,
and exactly one exchange per step - the sum of the flat LoRA-gradient bucket (plus one scalar:
the global count of scored tokens, so every rank scales its loss gradient by 1/n_global and the
summed bucket IS the global-batch mean gradient).  On GPUs the exchange goes through the C ABI
(mft_comm_init / mft_allreduce_sum_f32 / mft_allreduce_sum_i64 of include/mft_cuda.h: NCCL bound
by the kernel library itself, the calls a C++ host would make); torch.distributed only carries
the rendezvous (the 128-byte communicator id), barriers and the timing reduction.  CPU tests run
the same logic over gloo.  Nothing else crosses ranks."""
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
            dist.init_process_group("cpu:gloo,cuda:nccl" if self.backend == "nccl" else self.backend, rank=self.rank,
                                    world_size=self.size, timeout=timeout, **kw)
        self._abi_comm = False
        if self.size > 1 and self.backend == "nccl":
            self._init_abi_comm()

    def _init_abi_comm(self):
        """Create the kernel library's own communicator: rank 0 makes the id, the host-side group hands it round."""
        import ctypes as C

        from . import _lib as L
        L.init(self.local_rank)
        ident = (C.c_uint8 * 128)()
        if self.rank == 0:
            L.call("mft_comm_unique_id", ident)
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=0, device=torch.device("cpu"))
        ident = (C.c_uint8 * 128).from_buffer_copy(box[0])
        L.call("mft_comm_init", self.rank, self.size, ident)
        self._abi_comm = True

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
            if self._abi_comm and t.is_cuda:
                from . import _lib as L
                assert t.dtype == torch.float32 and t.is_contiguous()
                L.call("mft_allreduce_sum_f32", t.data_ptr(), t.numel(), torch.cuda.current_stream().cuda_stream)
            else:
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
        if self._abi_comm:
            from . import _lib as L
            L.call("mft_allreduce_sum_i64", t.data_ptr(), 1, torch.cuda.current_stream().cuda_stream)
        else:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return int(t.item())

    def barrier(self):
        if self.size > 1:
            dist.barrier()

    def close(self):
        if self._abi_comm:
            from . import _lib as L
            torch.cuda.synchronize()
            L.call("mft_comm_destroy")
            self._abi_comm = False
        if self.size > 1 and dist.is_initialized():
            dist.destroy_process_group()
