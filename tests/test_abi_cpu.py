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


def test_tile_plan_of_the_pair_gemm_on_the_benchmark_shapes(lib):
    """Host logic only (no launch): which tile the CTA-pair GEMM takes for the linear layers of the Gemma-3-1B step at
    16384 tokens.  Without a device the plan assumes 148 SMs, the part this build targets."""
    import torch
    if torch.cuda.is_available() and torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the expectations below are for 148 SMs")
    fn = lib.mft_gemm_nt_tile_cols
    fn.restype = ctypes.c_int32
    fn.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)]
    BF16, F32 = 1, 0

    def cols(m, n, k, k2=0, dt=BF16):
        out = ctypes.c_int32(-1)
        assert fn(m, n, k, k2, dt, ctypes.byref(out)) == 0
        return out.value

    T = 16384
    # bf16 outputs whose width is 384 * j: down projection, gate|up dX, q|k|v, attention output, q|k|v dX, gate|up
    for n, k, k2 in [(1152, 6912, 16), (1152, 13824, 32), (1536, 1152, 48), (1152, 1024, 16), (1152, 1536, 48), (13824, 1152, 32)]:
        assert cols(T, n, k, k2) == 384, (n, k)
    assert cols(T, 1024, 1152, 16) == 256             # three 384-wide tiles would cover 1152 columns for 1024
    assert cols(T, 640, 2048, 8) == 384               # ragged last tile (Gemma-3-270M's hidden width)
    assert cols(T, 1152, 262144, 0, F32) == 384       # lm-head dHidden: f32, K split, long K ranges
    assert cols(T, 1152, 1152, 0, F32) == 256         # f32 under a short K: the streaming epilogue is not overlapped
    assert cols(512, 384, 4096) == 256                # two tiles: one wave either way, and the wide wave is the longer one
    assert cols(4096, 896, 4864) == 256               # Qwen2.5-0.5B's down projection at 4096 tokens: one wave of tiles either way
    assert cols(128, 1152, 6912) == 0 and cols(T, 128, 6912) == 0     # below 256 rows / 192 columns another kernel runs
    assert fn(0, 1152, 1152, 0, BF16, ctypes.byref(ctypes.c_int32())) != 0


def test_product_does_not_import_the_oracle():
    for path in list((ROOT / "mobilefinetuner_b200").rglob("*.py")) + list((ROOT / "mobilefinetuner_b200").rglob("*.c*")):
        text = path.read_text(errors="ignore")
        assert "oracle" not in text.replace("oracle/", "oracle/") or "import oracle" not in text and "from oracle" not in text, path
