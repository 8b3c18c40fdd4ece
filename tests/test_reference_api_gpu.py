"""GPU suite: the reference's OWN unit tests for the step's path (analytic attention / softmax /
repeat-kv / RMSNorm / RoPE / cross-entropy / LoRA-merge / leaf-accumulation answers), compiled
unchanged against this repo's C++ operator API (mobilefinetuner_b200/operator, namespace ops) and
linked with libmft_operators.so -> libmft_cuda.so, so every operator they call runs as CUDA kernels.
The executables are built by `make -C oracle api_tests` where the reference tree is mounted and
travel with the repo; their sources are never copied into it."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
BIN = ROOT / "oracle" / "_ref" / "api_tests"
NAMES = ["test_qkt_softmax_grad", "test_repeat_kv_softmax_grad", "test_attention_single_layer_backward", "test_rmsnorm_unit",
         "test_apply_rope_layout", "test_autograd_leaf_accum", "test_selected_token_lm_loss", "test_memory_efficient_attention_grad",
         "test_lora_linear", "test_tensor_slice"]


@pytest.mark.parametrize("name", NAMES)
def test_reference_unit_test_passes_on_gpu(name):
    from parity import require_built
    exe = require_built(BIN / name, "the reference unit test compiled against this repository's operator API")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, f"{name} failed:\n{r.stdout[-3000:]}\n{r.stderr[-2000:]}"
