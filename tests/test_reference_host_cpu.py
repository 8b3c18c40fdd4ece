"""CPU suite: the reference's own host-side unit tests that need no outside files, compiled UNCHANGED together with
the reference's dataset / tokenizer sources against this repository's ops::Tensor and ModelRegistry through the
`operators` CMake target (`make -C oracle host_tests`):
  * data/test_jsonl_mask_alignment.cpp - the data format on the input side of the fine-tuning step: JSONL records become
    padded int32 id / label tensors with masked labels and a float attention mask;
  * core/test_tokenizer_factory.cpp - which tokenizer a model directory selects.
Host-only: no GPU is touched."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
BIN = ROOT / "oracle" / "_ref" / "host_tests"


@pytest.mark.parametrize("name", ["test_jsonl_mask_alignment", "test_tokenizer_factory"])
def test_reference_host_unit_test_passes_against_this_api(tmp_path, name):
    EXE = BIN / name
    ref = Path(os.environ.get("MFT_REFERENCE", "/root/reference"))
    if not EXE.exists():
        if not (ref / "operator" / "finetune_ops" / "data" / "wikitext2_dataset.cpp").exists():
            pytest.skip("neither the built test nor the reference's sources are present on this machine")
        r = subprocess.run(["make", "-C", str(ROOT / "oracle"), f"REF={ref}", "host_tests"], capture_output=True, text=True, timeout=1200)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    env = dict(os.environ, LD_LIBRARY_PATH=str(ROOT / "mobilefinetuner_b200") + ":" + os.environ.get("LD_LIBRARY_PATH", ""), TMPDIR=str(tmp_path))
    r = subprocess.run([str(EXE)], capture_output=True, text=True, timeout=120, env=env, cwd=tmp_path)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
