"""CPU suite: host logic of the step driver.  The learning-rate schedule of the reference's trainers (get_lr) is
pure host arithmetic inside libmft_cuda.so; it is compared with the restatement for every optimizer step of
several runs, including the integer truncation of the warm-up length."""
import ctypes as C

import pytest

from oracle import restate as R


@pytest.mark.parametrize("scheduler", ["linear", "cosine", "constant"])
@pytest.mark.parametrize("total,warmup", [(1, 0.03), (33, 0.03), (34, 0.03), (100, 0.1), (1000, 0.0), (7, 0.5)])
def test_learning_rate_schedule_matches_the_trainers(scheduler, total, warmup):
    from mobilefinetuner_b200 import _lib as L
    cfg = L.TrainerConfig(2e-4, 0.0, 0.9, 0.999, 1e-8, 1.0, warmup, L.LR_SCHEDULERS[scheduler], 1, total)
    for step in list(range(1, min(total, 60) + 2)) + [total, total + 5]:
        got = L.call("mft_trainer_lr", C.byref(cfg), step)
        want = R.trainer_lr(step, 2e-4, warmup, scheduler, total)
        assert abs(got - want) <= 1e-6 * 2e-4 + 1e-12, (step, got, want)


def test_total_updates_formula_of_the_wrapper():
    """ceil(ceil(num_sequences / micro_batch) * epochs / grad_accum), at least 1 (both trainers)."""
    from mobilefinetuner_b200.engine import LoraTrainer

    class FakeEngine:
        _h = None

    import mobilefinetuner_b200._lib as L
    made = {}
    orig = L.call
    def fake_call(name, *args):
        if name == "mft_trainer_create":
            made["cfg"] = args[1]._obj
            return 0
        return orig(name, *args)
    L.call = fake_call
    try:
        LoraTrainer(FakeEngine(), num_sequences=1001, micro_batch_size=4, num_epochs=3, grad_accum_steps=8)
    finally:
        L.call = orig
    assert made["cfg"].total_updates == (251 * 3 + 7) // 8
    assert made["cfg"].grad_accum_steps == 8


def test_perplexity_result_matches_the_reference_aggregation():
    """mft_ppl_result is host arithmetic: sum of loss * count in double, float mean, expf."""
    import numpy as np
    from mobilefinetuner_b200 import _lib as L
    g = np.random.Generator(np.random.PCG64(5))
    losses = g.uniform(2.0, 11.0, 7).astype(np.float32)
    labels = [np.where(g.random((3, 40)) < 0.2, -100, 5).astype(np.int32) for _ in losses]
    acc = L.PplAccum(0.0, 0, 0)
    for loss, lab in zip(losses, labels):          # what mft_model_eval_ppl_batch adds per batch
        valid = int((lab != -100).sum())
        acc.sum_loss += float(np.float32(loss) * np.float32(valid))
        acc.sum_tokens += valid
        acc.n_batches += 1
    nll, ppl = C.c_float(), C.c_float()
    L.call("mft_ppl_result", C.byref(acc), C.byref(nll), C.byref(ppl))
    w_nll, w_ppl, w_tokens = R.ppl_accumulate(losses, labels)
    assert acc.sum_tokens == w_tokens
    assert abs(nll.value - w_nll) <= 1e-6 * w_nll and abs(ppl.value - w_ppl) <= 2e-6 * w_ppl
    empty = L.PplAccum(0.0, 0, 0)
    L.call("mft_ppl_result", C.byref(empty), C.byref(nll), C.byref(ppl))
    assert nll.value == 0.0 and ppl.value == 1.0
