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
