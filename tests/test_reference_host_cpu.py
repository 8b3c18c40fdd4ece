"""CPU suite: the reference's own dataset unit test (data/test_jsonl_mask_alignment.cpp) compiled UNCHANGED, together
with the reference's dataset source, against this repository's ops::Tensor through the `operators` CMake target
(`make -C oracle host_tests`).  It checks the data format on the input side of the fine-tuning step: JSONL records
become padded int32 id / label tensors with masked labels and a float attention mask.  Host-only: no GPU is touched."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
EXE = ROOT / "oracle" / "_ref" / "host_tests" / "test_jsonl_mask_alignment"


def test_reference_dataset_unit_test_passes_against_this_tensor(tmp_path):
    ref = Path(os.environ.get("MFT_REFERENCE", "/root/reference"))
    if not EXE.exists():
        if not (ref / "operator" / "finetune_ops" / "data" / "wikitext2_dataset.cpp").exists():
            pytest.skip("neither the built test nor the reference's sources are present on this machine")
        r = subprocess.run(["make", "-C", str(ROOT / "oracle"), f"REF={ref}", "host_tests"], capture_output=True, text=True, timeout=1200)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    env = dict(os.environ, LD_LIBRARY_PATH=str(ROOT / "mobilefinetuner_b200") + ":" + os.environ.get("LD_LIBRARY_PATH", ""), TMPDIR=str(tmp_path))
    r = subprocess.run([str(EXE)], capture_output=True, text=True, timeout=120, env=env, cwd=tmp_path)
    assert r.returncode == 0 and "test passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
