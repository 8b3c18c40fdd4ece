"""GPU suite for the runtime part of the C ABI: the stream-ordered caching allocator (the device analogue of
MemoryManager / MemoryPool, operator/finetune_ops/core/memory_manager.cpp:34-145) and the data-parallel exchange
(mft_comm_*).  The two-rank cases start one child process per GPU and are skipped on a single-GPU box."""
import ctypes as C
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _stats(L):
    s = (C.c_int64 * 6)()
    L.call("mft_mem_stats", s)
    return dict(in_use=s[0], cached=s[1], peak=s[2], driver_allocs=s[3], reuses=s[4], cross_stream_waits=s[5])


def test_allocator_reuses_blocks_and_reports_statistics():
    import torch
    from mobilefinetuner_b200 import _lib as L
    L.init(0)
    torch.cuda.synchronize()
    L.call("mft_empty_cache")
    st = torch.cuda.current_stream().cuda_stream
    base = _stats(L)
    assert base["cached"] == 0
    p, q = C.c_void_p(), C.c_void_p()
    L.call("mft_malloc", 3_000_000, st, C.byref(p))             # rounds up to 2 MiB granularity: 4 MiB
    a = _stats(L)
    assert a["in_use"] - base["in_use"] == 4 << 20 and a["driver_allocs"] == base["driver_allocs"] + 1
    L.call("mft_free", p, st)
    b = _stats(L)
    assert b["in_use"] == base["in_use"] and b["cached"] == 4 << 20
    L.call("mft_malloc", 3_500_000, st, C.byref(q))             # same size class: served from the cache, same block
    c = _stats(L)
    assert q.value == p.value and c["driver_allocs"] == a["driver_allocs"] and c["reuses"] == b["reuses"] + 1 and c["cached"] == 0
    small = [C.c_void_p() for _ in range(3)]
    for h in small:
        L.call("mft_malloc", 1000, st, C.byref(h))              # 512-byte granularity below 1 MiB: 1024 each
    assert _stats(L)["in_use"] - c["in_use"] == 3 * 1024 and len({h.value for h in small}) == 3
    for h in small:
        L.call("mft_free", h, st)
    L.call("mft_free", q, st)
    d = _stats(L)
    assert d["cached"] == (4 << 20) + 3 * 1024 and d["peak"] >= c["in_use"]
    L.call("mft_trim_cache", 2048)                                # largest blocks go first, 2 KiB may stay
    e = _stats(L)
    assert e["cached"] == 2048
    L.call("mft_empty_cache")
    assert _stats(L)["cached"] == 0
    with pytest.raises(L.MftError):
        L.call("mft_free", C.c_void_p(0xdead000), st)            # a pointer the allocator never handed out


def test_allocator_orders_reuse_across_streams():
    """A block freed on stream A while A still has writes to it queued, then requested on stream B: B's first write
    must land after A's last one (the allocator makes B wait on the release event; the host is never blocked)."""
    import torch
    from mobilefinetuner_b200 import _lib as L
    L.init(0)
    torch.cuda.synchronize()
    L.call("mft_empty_cache")
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    n = 256 << 20
    before = _stats(L)
    p, q = C.c_void_p(), C.c_void_p()
    L.call("mft_malloc", n, sa.cuda_stream, C.byref(p))
    for _ in range(40):                                           # ~10 GB of queued writes on A
        L.call("mft_memset", p, 1, n, sa.cuda_stream)
    L.call("mft_free", p, sa.cuda_stream)
    L.call("mft_malloc", n, sb.cuda_stream, C.byref(q))
    assert q.value == p.value
    L.call("mft_memset", q, 2, n, sb.cuda_stream)
    after = _stats(L)
    assert after["reuses"] == before["reuses"] + 1
    assert after["cross_stream_waits"] == before["cross_stream_waits"] + 1     # A's queue cannot have drained yet
    host = np.empty(1 << 20, np.uint8)
    L.call("mft_memcpy_d2h", host.ctypes.data, q.value + n - host.size, host.size, sb.cuda_stream)
    torch.cuda.synchronize()
    assert (host == 2).all()
    L.call("mft_free", q, sb.cuda_stream)
    # same stream: no wait is needed, stream order already covers it
    L.call("mft_malloc", n, sb.cuda_stream, C.byref(p))
    assert _stats(L)["cross_stream_waits"] == after["cross_stream_waits"]
    L.call("mft_free", p, sb.cuda_stream)
    torch.cuda.synchronize()
    L.call("mft_empty_cache")


def test_single_rank_communicator_is_a_no_op():
    import torch
    from mobilefinetuner_b200 import _lib as L
    L.init(0)
    L.call("mft_comm_destroy")
    L.call("mft_comm_init", 0, 1, None)
    t = torch.arange(8, dtype=torch.float32, device="cuda")
    L.call("mft_allreduce_sum_f32", t.data_ptr(), t.numel(), torch.cuda.current_stream().cuda_stream)
    L.call("mft_comm_wait", torch.cuda.current_stream().cuda_stream, 5000)
    assert t.tolist() == list(range(8))
    r, w = C.c_int32(-1), C.c_int32(-1)
    L.call("mft_comm_info", C.byref(r), C.byref(w), None)
    assert (r.value, w.value) == (0, 1)
    code = C.c_int32(7)
    L.call("mft_comm_async_error", C.byref(code))
    assert code.value == 0
    L.call("mft_comm_destroy")
    with pytest.raises(L.MftError):
        L.call("mft_comm_init", 2, 2, None)                       # rank outside the world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(mode, tmp_path, n=2):
    import torch
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MFT_DIST_TIMEOUT_S="60", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "comm_worker.py"), mode, str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


def test_two_ranks_through_the_abi_match_the_full_batch(tmp_path):
    """Sharded by sample over two GPUs, gradients summed by mft_allreduce_sum_f32: same loss, gradients and updated
    adapters as one GPU on the whole batch."""
    _run_ranks("step", tmp_path)
    full, r0, r1 = (np.load(tmp_path / f) for f in ("full.npz", "rank0.npz", "rank1.npz"))
    assert np.array_equal(r0["after"], r1["after"])               # replicas stay identical
    cos = float(r0["grad"].astype(np.float64) @ full["grad"].astype(np.float64) /
                (np.linalg.norm(r0["grad"]) * np.linalg.norm(full["grad"])))
    assert cos >= 0.99999
    assert abs(float(r0["loss"]) - float(full["loss"])) <= 1e-4 * abs(float(full["loss"]))
    assert int(r0["n_global"]) == int(full["n_global"])           # integer work: exact


def test_a_departed_rank_turns_into_a_status_not_a_hang(tmp_path):
    """Rank 1 leaves between steps (nothing in flight) and says so in a file; rank 0 reads it before its next launch,
    aborts the communicator and from then on gets MFT_ERR_NCCL from the exchange instead of queueing a collective
    that could never finish."""
    out = _run_ranks("depart", tmp_path)
    assert "rank 0: exchange refused after abort: MFT_ERR_NCCL" in out
