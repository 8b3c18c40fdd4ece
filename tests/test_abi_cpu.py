"""CPU suite: the C ABI library builds (nvcc cross-compiles sm_100a without a GPU), loads,
and exports every symbol that include/mft_cuda.h declares.  No compute calls here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from mobilefinetuner_b200 import build
    path = build.build()
    return ctypes.CDLL(str(path))


def declared_symbols():
    text = (ROOT / "include" / "mft_cuda.h").read_text() + (ROOT / "include" / "mft_step.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mft_[a-z0-9_]+)\s*\(", text)) - {"mft_model"})


def test_header_declares_the_path():
    names = declared_symbols()
    for required in ["mft_gemm_nt", "mft_gemm_tn_acc", "mft_attn_fwd", "mft_attn_bwd", "mft_lmhead_ce_fwd",
                     "mft_lmhead_ce_bwd", "mft_rmsnorm_fwd", "mft_layernorm_fwd", "mft_act_fwd", "mft_headnorm_rope_fwd",
                     "mft_embedding_gather", "mft_adam_step", "mft_malloc"]:
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert missing == []


def test_binding_signatures_cover_the_header():
    from mobilefinetuner_b200 import _lib
    assert sorted(_lib.exported_names()) == declared_symbols()
    assert _lib.missing_symbols() == []


def test_no_cpu_fallback_without_device(lib):
    """Without a CUDA device mft_init must fail loudly (status != 0 and a message), never fall back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib.mft_init.restype = ctypes.c_int32
    lib.mft_last_error.restype = ctypes.c_char_p
    assert lib.mft_init(0) != 0
    assert b"no CUDA device" in lib.mft_last_error()


def test_product_does_not_import_the_oracle():
    for path in list((ROOT / "mobilefinetuner_b200").rglob("*.py")) + list((ROOT / "mobilefinetuner_b200").rglob("*.c*")):
        text = path.read_text(errors="ignore")
        assert "oracle" not in text.replace("oracle/", "oracle/") or "import oracle" not in text and "from oracle" not in text, path
