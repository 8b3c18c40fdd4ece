"""CPU suite: pins oracle/restate.py (the numpy restatement of the reference's operators)
against tests/golden/ops_golden.npz, i.e. against outputs of the compiled reference itself.
fp32-vs-float64 accumulation noise only: tolerances are ~1e-5 relative."""
import numpy as np
import pytest

from conftest import rel_err
from oracle import restate as R

TOL = 2e-5


@pytest.mark.parametrize("name", ["attn_causal_gqa", "attn_window_rope", "attn_hd256_window", "attn_hd128"])
def test_attention_chain(golden, name):
    i, o, p = golden.case(name)
    out, dq, dk, dv = R.attention_fwd_bwd(i["q"], i["k"], i["v"], i["dO"], p["scale"], int(p["window"]), p["rope_theta"])
    assert rel_err(out, o["O"]) < TOL
    assert rel_err(dq, o["dQ"]) < TOL
    assert rel_err(dk, o["dK"]) < TOL
    assert rel_err(dv, o["dV"]) < TOL


def test_lora_linear(golden):
    i, o, p = golden.case("lora_linear")
    y = R.lora_linear_fwd(i["x"], i["W"], i["bias"], i["A"], i["B"], p["scale"])
    dx, dA, dB = R.lora_linear_bwd(i["x"], i["W"], i["A"], i["B"], p["scale"], i["dY"])
    assert rel_err(y, o["y"]) < TOL and rel_err(dx, o["dx"]) < TOL
    assert rel_err(dA, o["dA"]) < TOL and rel_err(dB, o["dB"]) < TOL


def test_matmul(golden):
    i, o, _ = golden.case("matmul")
    assert rel_err(R.matmul(i["a"], i["b"]), o["y"]) < TOL
    assert rel_err(R.matmul(i["dY"], i["b"].T), o["da"]) < TOL
    i, o, _ = golden.case("matmul_rhs_T")
    assert rel_err(R.matmul(i["a"], i["b"].T), o["y"]) < TOL
    assert rel_err(R.matmul(i["dY"], i["b"]), o["da"]) < TOL


@pytest.mark.parametrize("name,unit", [("rms_norm", True), ("rms_norm_affine", False)])
def test_rms_norm(golden, name, unit):
    i, o, p = golden.case(name)
    assert rel_err(R.rms_norm_fwd(i["x"], i["w"], p["eps"], unit), o["y"]) < TOL
    dx, dw = R.rms_norm_bwd(i["dY"], i["x"], i["w"], p["eps"], unit)
    assert rel_err(dx, o["dx"]) < TOL and rel_err(dw, o["dw"]) < TOL


def test_layer_norm(golden):
    i, o, p = golden.case("layer_norm")
    assert rel_err(R.layer_norm_fwd(i["x"], i["w"], i["b"], p["eps"]), o["y"]) < TOL
    dx, dw, db = R.layer_norm_bwd(i["dY"], i["x"], i["w"], p["eps"])
    assert rel_err(dx, o["dx"]) < 5e-5 and rel_err(dw, o["dw"]) < TOL and rel_err(db, o["db"]) < TOL


def test_activations(golden):
    i, o, _ = golden.case("gelu")
    assert rel_err(R.gelu_fwd(i["x"]), o["y"]) < TOL
    assert rel_err(i["dY"] * R.gelu_grad(i["x"]), o["dx"]) < TOL
    i, o, _ = golden.case("swiglu")
    assert rel_err(R.swiglu_fwd(i["gate"], i["up"]), o["y"]) < TOL
    dg, du = R.swiglu_bwd(i["dY"], i["gate"], i["up"])
    assert rel_err(dg, o["dgate"]) < TOL and rel_err(du, o["dup"]) < TOL
    i, o, _ = golden.case("geglu")
    assert rel_err(R.geglu_fwd(i["gate"], i["up"]), o["y"]) < TOL
    dg, du = R.geglu_bwd(i["dY"], i["gate"], i["up"])
    assert rel_err(dg, o["dgate"]) < TOL and rel_err(du, o["dup"]) < TOL


@pytest.mark.parametrize("name", ["rope_1e4", "rope_1e6"])
def test_rope(golden, name):
    i, o, p = golden.case(name)
    assert rel_err(R.rope_fwd(i["x"], p["rope_theta"]), o["y"]) < TOL
    assert rel_err(R.rope_bwd(i["dY"], p["rope_theta"]), o["dx"]) < TOL
    # position 0 is the identity (core/test_apply_rope_layout.cpp)
    assert np.array_equal(R.rope_fwd(i["x"], p["rope_theta"])[:, :, 0], i["x"][:, :, 0])


def test_repeat_kv_bit_exact(golden):
    i, o, p = golden.case("repeat_kv")
    assert np.array_equal(R.repeat_kv(i["x"], int(p["repeat"])), o["y"])
    assert rel_err(R.repeat_kv_bwd(i["dY"], int(p["repeat"])), o["dx"]) < 1e-6


def test_lm_cross_entropy(golden):
    i, o, _ = golden.case("lm_ce")
    loss, dlogits, n = R.lm_cross_entropy(i["logits"], i["labels"])
    assert n == int((i["labels"][:, 1:] != -100).sum())
    assert abs(loss - o["loss"][0]) < 1e-5 * abs(o["loss"][0])
    assert rel_err(dlogits, o["dlogits"]) < TOL
    assert np.all(dlogits[:, -1, :] == 0)


def test_lm_head_ce_dense_equals_streaming(golden):
    i, o, _ = golden.case("lm_head_ce")
    loss, dh = R.lm_head_ce(i["hidden"], i["W"], i["labels"])
    assert abs(loss - o["loss"][0]) < 1e-5 * abs(o["loss"][0])
    assert rel_err(dh, o["dhidden"]) < TOL
    _, os_, _ = golden.case("streaming_ce")
    assert abs(os_["loss"][0] - o["loss"][0]) < 1e-5 and rel_err(os_["dhidden"], o["dhidden"]) < 1e-4


def test_lm_ce_all_ignored_is_nan_with_zero_grad(golden):
    i, o, _ = golden.case("lm_ce_all_ignored")
    assert np.isnan(o["loss"][0])
    loss, dh = R.lm_head_ce(i["hidden"], i["W"], i["labels"])
    assert np.isnan(loss) and np.all(dh == 0)


def test_label_out_of_range_raises():
    with pytest.raises(IndexError):
        R.lm_cross_entropy(np.zeros((1, 3, 4), np.float32), np.array([[0, 4, 1]], np.int32))


@pytest.mark.parametrize("name", ["adam_clip", "adam_wd"])
def test_adam(golden, name):
    i, o, p = golden.case(name)
    pp, m, v = i["p"], np.zeros_like(i["p"]), np.zeros_like(i["p"])
    for step in range(int(p["steps"])):
        g = i[f"g{step}"]
        g = g * R.clip_scale([g], p.get("max_grad_norm", 0.0))
        pp, m, v = R.adam_step(pp, g, m, v, step + 1, p["lr"], weight_decay=p.get("weight_decay", 0.0))
    assert rel_err(pp, o["p"]) < 1e-6


def test_bf16_round_is_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 1e-40, 65504.0], np.float32)
    import torch
    assert np.array_equal(R.bf16_round(x), torch.from_numpy(x).bfloat16().float().numpy())
