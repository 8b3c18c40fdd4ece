"""GPU parity suite at the benchmark configurations' own sizes, against the compiled reference run live on this
machine's host cores (oracle/_ref):

  * GPT-2 small at full size (12 layers, 768 wide, vocabulary 50257, batch 4 x 128, r = 8 on c_attn + c_proj),
    including the reference's rule that c_attn adapters receive no gradient;
  * the operator-level causal GQA attention sweep shape (14 query heads on 2 KV heads, head_dim 64) at S = 1024 with
    the full batch of 8, S = 2048 with batch 2 and S = 4096 with batch 1 (the dense CPU chain needs S*S floats per
    head), driven like optim/test_attention_single_layer_backward.cpp:82-116: O, dQ, dK, dV;
  * Qwen2.5-0.5B widths (hidden 896, 14/2 heads of 64, SwiGLU 4864, q/k/v bias, full vocabulary 151936, r = 16 on
    q,k,v,o) on a 2-layer stack, 2 x 512 tokens;
  * Gemma-3-270M widths (hidden 640, 4/1 heads of 256, GeGLU 2048, full vocabulary 262144, r = 8 with alpha 32 on all
    seven linears) on a sliding + global layer pair, 1 x 640 tokens so that the 512-token window is active.

Tolerances are the path's: loss relative error <= 2e-3, LoRA-gradient cosine >= 0.999, updated parameters within
2e-2 (tests/parity.py); attention outputs cosine >= 0.999 and max-norm relative error <= 2e-2."""
import numpy as np
import pytest

from conftest import cosine, rel_err
from parity import check, require_reference, run_engine

pytestmark = pytest.mark.gpu


def _model_case(spec, batch, seq, seeds):
    from mobilefinetuner_b200 import synth
    params = synth.make_params(spec, seeds[0], 0.05)
    lora = synth.make_lora(spec, seeds[1])
    data = synth.make_batch(spec, batch, seq, seeds[2])
    return dict(spec=spec, batch=batch, seq=seq, seeds=seeds, norm_jitter=0.05, params=params, lora=lora, batch_data=data)


def _against_live_reference(case):
    from model_cases import STEP
    from oracle import model_case
    require_reference()
    ids, labels = case["batch_data"]
    ref = model_case.run_reference_step(case["spec"], case["params"], case["lora"], ids, labels, **STEP)
    loss, grads, after, lora0 = run_engine(case)
    worst = check(loss, grads, after, lora0, float(ref["loss"][0]), ref["grads"], ref["lora_after"])
    print("reference:", ref["timing"].strip().replace("\n", " | "), "| worst gradient cosine", worst)
    return ref, grads


def test_gpt2_small_full_size_step():
    from mobilefinetuner_b200 import configs as Cf
    case = _model_case(Cf.GPT2_SMALL, 4, 128, (1101, 1102, 1103))
    ref, grads = _against_live_reference(case)
    # c_attn A, B, c_proj A, B per layer: the QKV split severs autograd, only c_proj adapters get gradients
    have = [g is not None for g in ref["grads"]]
    assert have == [False, False, True, True] * 12
    assert [g is not None for g in grads] == have


def test_qwen25_05b_widths_step():
    from mobilefinetuner_b200 import configs as Cf
    spec = Cf.reduced(Cf.QWEN25_05B, layers=2)
    assert (spec.hidden, spec.inter, spec.vocab, spec.n_heads, spec.n_kv_heads, spec.lora_rank) == (896, 4864, 151936, 14, 2, 16)
    _against_live_reference(_model_case(spec, 2, 512, (1301, 1302, 1303)))


def test_gemma3_270m_widths_step():
    from mobilefinetuner_b200 import configs as Cf
    spec = Cf.reduced(Cf.GEMMA3_270M, layers=2, global_every=2)
    assert (spec.hidden, spec.inter, spec.vocab, spec.head_dim, spec.lora_rank, spec.lora_alpha) == (640, 2048, 262144, 256, 8, 32.0)
    assert spec.layer_is_sliding(0) and not spec.layer_is_sliding(1) and spec.sliding_window == 512
    _against_live_reference(_model_case(spec, 1, 640, (1401, 1402, 1403)))


@pytest.mark.parametrize("S,B", [(1024, 8), (2048, 2), (4096, 1)])
def test_attention_sweep_shape_against_live_reference(S, B):
    import torch
    from mobilefinetuner_b200 import ops as O
    from oracle import refrun
    from oracle import restate as R
    require_reference()
    g = np.random.Generator(np.random.PCG64(4000 + S))
    nh, nkv, hd = 14, 2, 64
    q, k, v, dO = (R.bf16_round(g.standard_normal(s).astype(np.float32)) for s in [(B, nh, S, hd), (B, nkv, S, hd), (B, nkv, S, hd), (B, nh, S, hd)])
    ref = refrun.run_op("attention", {"q": q, "k": k, "v": v, "dO": dO}, scale=0.125, window=0)

    def dev(x):          # [B, h, S, hd] view over token-major storage, the layout the step uses
        return torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 1, 3))).cuda().bfloat16().permute(0, 2, 1, 3)
    qd, kd, vd, dod = dev(q), dev(k), dev(v), dev(dO)
    o, lse = O.attention_fwd(qd, kd, vd, 0.125, 0)
    dq, dk, dv = O.attention_bwd(qd, kd, vd, o, dod, lse, 0.125, 0)
    for name, got, want in [("O", o, ref["O"]), ("dQ", dq, ref["dQ"]), ("dK", dk, ref["dK"]), ("dV", dv, ref["dV"])]:
        got = got.float().cpu().numpy()
        assert np.isfinite(got).all()
        c, e = cosine(got, want), rel_err(got, want)
        print(f"S={S} {name}: cosine {c:.6f} max-norm rel err {e:.4f}")
        assert c >= 0.999 and e <= 2e-2, (name, c, e)
    assert O.device_status() == 0
