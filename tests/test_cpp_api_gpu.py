"""GPU suite: the C++ operator API's step driver (ops::AutoModelForCausalLM + ops::AutoTrainer, the same calls the
reference's graph/test_auto_model.cpp makes) against the reference's committed outputs.  A small C++ program
(tests/cpp/auto_trainer_step.cpp, built by mobilefinetuner_b200.build) runs one step on the reduced model cases
and dumps loss, LoRA gradients and updated LoRA tensors."""
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from model_cases import CASES, STEP
from parity import check

pytestmark = pytest.mark.gpu
EXE = ROOT / "mobilefinetuner_b200" / "csrc" / "build" / "auto_trainer_step"


@pytest.mark.parametrize("name", ["gemma_tiny", "qwen_tiny", "gpt2_tiny"])
def test_cpp_auto_trainer_step_matches_reference(tmp_path, name):
    assert EXE.exists(), "auto_trainer_step was not built (python -m mobilefinetuner_b200.build)"
    from mobilefinetuner_b200 import synth
    case = CASES[name]
    spec = case["spec"]
    params = synth.make_params(spec, case["seeds"][0], case["norm_jitter"])
    lora = synth.make_lora(spec, case["seeds"][1])
    ids, labels = synth.make_batch(spec, case["batch"], case["seq"], case["seeds"][2])
    (tmp_path / "params").mkdir()
    (tmp_path / "lora").mkdir()
    (tmp_path / "config.json").write_text(spec.config_json())
    (tmp_path / "case.txt").write_text(f"batch {case['batch']}\nseq {case['seq']}\nlr {STEP['lr']}\nmax_grad_norm {STEP['max_grad_norm']}\n"
                                        f"lora_rank {spec.lora_rank}\nlora_alpha {spec.lora_alpha}\nlora_targets {','.join(spec.lora_targets)}\n")
    for i, a in enumerate(params):
        np.ascontiguousarray(a, np.float32).tofile(tmp_path / "params" / f"{i:04d}.bin")
    for i, a in enumerate(lora):
        np.ascontiguousarray(a, np.float32).tofile(tmp_path / "lora" / f"{i:04d}.bin")
    np.ascontiguousarray(ids, np.int32).tofile(tmp_path / "ids.bin")
    np.ascontiguousarray(labels, np.int32).tofile(tmp_path / "labels.bin")
    r = subprocess.run([str(EXE), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    out = tmp_path / "out"
    loss = float(np.fromfile(out / "loss.bin", np.float32)[0])
    grads = [np.fromfile(out / f"grad_{i:04d}.bin", np.float32).reshape(a.shape) if (out / f"grad_{i:04d}.bin").exists() else None
             for i, a in enumerate(lora)]
    after = [np.fromfile(out / f"lora_{i:04d}.bin", np.float32).reshape(a.shape) for i, a in enumerate(lora)]
    z = np.load(ROOT / "tests" / "golden" / "model_golden.npz")
    ref_grads = [z[f"{name}/grad/{i}"] if f"{name}/grad/{i}" in z.files else None for i in range(len(lora))]
    ref_after = [z[f"{name}/after/{i}"] for i in range(len(lora))]
    check(loss, grads, after, lora, float(z[f"{name}/loss"][0]), ref_grads, ref_after)


def test_eager_operators_bf16_compute_type_matches_fp32():
    """ops::set_compute_dtype(kBFloat16) routes matmul / LoRALinear / memory_efficient_attention / the streaming lm-head
    loss to the tensor-core kernels; values and gradients must agree with the fp32 operators to bf16 rounding
    (tests/cpp/compute_dtype.cpp prints and checks cosine >= 0.999 and max error <= 2e-2 of the largest magnitude)."""
    exe = EXE.parent / "compute_dtype"
    assert exe.exists(), "compute_dtype was not built (python -c 'import __graft_entry__ as g; g.build()')"
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ALL OK" in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]
