"""CPU suite for the data-parallel plumbing (world size 2, gloo): sharding by sample, the global
scored-token count and the single sum-all-reduce of the gradient bucket.  With every rank scaling
its per-token terms by 1/n_global, the reduced bucket must equal the single-process global-batch
mean - the property the GPU step relies on."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from mobilefinetuner_b200.dist import World
    w = World("gloo")
    g = np.random.Generator(np.random.PCG64(5))
    labels = g.integers(0, 50, size=(8, 12)).astype(np.int32)
    labels[1, 3:7] = -100
    labels[6, 1:] = -100
    feats = g.standard_normal((8, 12, 16)).astype(np.float32)
    sl = w.shard(labels.shape[0])
    n_global = w.global_valid_count(labels[sl])
    valid = (labels[sl][:, 1:] != -100)[..., None]
    bucket = torch.from_numpy((feats[sl][:, :-1] * valid).sum(axis=(0, 1)) / n_global)     # local sum scaled by 1/n_global
    w.all_reduce_sum(bucket)
    t_max = w.all_reduce_max(float(rank + 1))
    np.save(os.path.join(out_dir, f"r{rank}.npy"), np.concatenate([bucket.numpy(), [n_global, t_max, sl.start, sl.stop]]))
    w.barrier()
    w.close()


def test_two_rank_bucket_equals_global_mean(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    g = np.random.Generator(np.random.PCG64(5))
    labels = g.integers(0, 50, size=(8, 12)).astype(np.int32)
    labels[1, 3:7] = -100
    labels[6, 1:] = -100
    feats = g.standard_normal((8, 12, 16)).astype(np.float32)
    valid = (labels[:, 1:] != -100)
    want = (feats[:, :-1] * valid[..., None]).sum(axis=(0, 1)) / valid.sum()
    r0, r1 = np.load(tmp_path / "r0.npy"), np.load(tmp_path / "r1.npy")
    assert np.allclose(r0[:16], want, rtol=1e-5, atol=1e-6) and np.array_equal(r0[:16], r1[:16])
    assert r0[16] == valid.sum() == r1[16]            # the count is integer work: exact
    assert r0[17] == 2.0 and r1[17] == 2.0            # max over ranks
    assert (r0[18], r0[19], r1[18], r1[19]) == (0, 4, 4, 8)


def test_single_process_world_is_a_no_op():
    sys.path.insert(0, str(ROOT))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    from mobilefinetuner_b200.dist import World
    w = World("gloo")
    assert w.size == 1 and w.shard(6) == slice(0, 6)
    t = torch.ones(3)
    assert torch.equal(w.all_reduce_sum(t), torch.ones(3))
    assert w.global_valid_count(np.array([[1, 2, -100, 4]])) == 2
    with pytest.raises(ValueError):
        World("gloo").__class__.shard(type("W", (), {"size": 4, "rank": 0})(), 6)
