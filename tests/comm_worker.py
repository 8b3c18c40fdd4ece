"""One rank of the two-GPU cases of tests/test_runtime_gpu.py (started by torch.distributed.run, one process per
GPU).  Modes:
  step    a LoRA step sharded by sample, gradients summed through mft_allreduce_sum_f32, next to the same step on
          the whole batch computed by rank 0 alone; results are written to <out>/rank{r}.npz and <out>/full.npz.
  depart  rank 1 leaves between steps with nothing in flight and leaves a note; rank 0 reads the note before its next
          launch, aborts the communicator and checks that the exchange is refused with a status.
"""
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from mobilefinetuner_b200 import _lib as L, synth  # noqa: E402
from mobilefinetuner_b200.configs import StepConfig  # noqa: E402
from mobilefinetuner_b200.dist import World  # noqa: E402
from mobilefinetuner_b200.engine import LoraStepEngine  # noqa: E402
from model_cases import CASES  # noqa: E402


def make_engine(spec, batch, seq, device):
    eng = LoraStepEngine(spec, batch, seq, device=device)
    eng.set_params(synth.make_params(spec, 1, 0.1))
    eng.set_lora(synth.make_lora(spec, 2))
    return eng


def mode_step(world, out):
    case = CASES["gemma_tiny"]
    spec, S = case["spec"], case["seq"]
    B = 4
    ids, labels = synth.make_batch(spec, B, S, 3)
    labels = labels.copy()
    labels[1, S // 2:] = -100                          # ranks score different numbers of tokens
    cfg = StepConfig("two_rank_case", spec, B, S, lr=2e-4, max_grad_norm=1.0)
    sl = world.shard(B)
    eng = make_engine(spec, B, S, world.local_rank)
    n_global = world.global_valid_count(labels[sl])
    loss, n_local = eng.forward_backward(ids[sl], labels[sl], n_global)
    world.all_reduce_sum(eng.grad_bucket())
    grad = eng.grad_bucket().cpu().numpy().copy()
    eng.optimizer_step(cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.max_grad_norm, 0.0)
    t = torch.tensor([loss * n_local / n_global], dtype=torch.float32, device="cuda")
    world.all_reduce_sum(t)                            # global mean loss = count-weighted mean of the local means
    np.savez(out / f"rank{world.rank}.npz", grad=grad, after=eng.param_bucket().cpu().numpy(), loss=float(t.item()), n_global=n_global)
    eng.close()
    if world.rank == 0:
        full = make_engine(spec, B, S, world.local_rank)
        loss_f, n_f = full.forward_backward(ids, labels)
        np.savez(out / "full.npz", grad=full.grad_bucket().cpu().numpy(), loss=loss_f, n_global=n_f)
        full.close()
    world.barrier()


def mode_depart(world, out):
    note = out / "rank1.left"
    t = torch.ones(1024, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):                                 # two healthy steps
        world.all_reduce_sum(t)
        L.call("mft_comm_wait", st, 30000)
    assert float(t[0].item()) == float(world.size ** 2)
    world.barrier()
    if world.rank == 1:
        torch.cuda.synchronize()                       # nothing of this rank is in flight
        note.write_text("left after step 2")
        return                                          # leaves without taking part in step 3
    deadline = time.time() + 30
    while not note.exists() and time.time() < deadline:
        time.sleep(0.05)
    assert note.exists(), "rank 1 never announced its departure"
    L.call("mft_comm_abort")                           # learned on the host, before the next launch
    try:
        world.all_reduce_sum(t)
    except L.MftError as e:
        assert "status -4" in str(e), e                # MFT_ERR_NCCL
        print("rank 0: exchange refused after abort: MFT_ERR_NCCL", flush=True)
    else:
        raise AssertionError("the exchange was queued on an aborted communicator")
    try:
        L.call("mft_comm_async_error", None)
    except L.MftError:
        pass
    else:
        raise AssertionError("mft_comm_async_error does not report the abort")
    world._abi_comm = False                            # nothing left to destroy
    L.call("mft_comm_destroy")


def main():
    mode, out = sys.argv[1], Path(sys.argv[2])
    world = World()
    assert world.size == 2 and world._abi_comm
    if mode == "step":
        mode_step(world, out)
        world.close()
    else:
        mode_depart(world, out)
        # the host-side group is not torn down collectively here: one side is already gone
    print(f"rank {world.rank}: done", flush=True)


if __name__ == "__main__":
    main()
