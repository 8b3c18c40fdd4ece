"""GPU parity suite, whole-model level: one LoRA fine-tuning step (forward + shifted cross
entropy + backward + clip + Adam) of the CUDA engine against the compiled reference on the
same seeded parameters and batch.  Checked against the committed reference outputs
(tests/golden/model_golden.npz) and, where oracle/_ref is present, against a fresh run of the
reference driver at a larger shape.  Tolerances are the path's: loss relative error <= 2e-3,
per-tensor LoRA-gradient cosine >= 0.999, and after one optimizer step per-element
|p' - p'_ref| <= 2e-2 * max(|p'_ref|, lr)."""
import numpy as np
import pytest

from conftest import ROOT, cosine
from model_cases import CASES, STEP

pytestmark = pytest.mark.gpu

LOSS_REL, GRAD_COS, STEP_REL = 2e-3, 0.999, 2e-2


@pytest.fixture(scope="module")
def model_golden():
    return np.load(ROOT / "tests" / "golden" / "model_golden.npz")


from parity import check, require_reference, run_engine  # noqa: E402


@pytest.mark.parametrize("name", list(CASES))
def test_step_matches_reference_golden(model_golden, name):
    case = CASES[name]
    loss, grads, after, lora0 = run_engine(case)
    n = len(lora0)
    ref_grads = [model_golden[f"{name}/grad/{i}"] if f"{name}/grad/{i}" in model_golden.files else None for i in range(n)]
    ref_after = [model_golden[f"{name}/after/{i}"] for i in range(n)]
    check(loss, grads, after, lora0, float(model_golden[f"{name}/loss"][0]), ref_grads, ref_after)


def test_gpt2_reference_gives_no_gradient_to_c_attn(model_golden):
    """The reference's QKV split severs autograd: c_attn LoRA tensors have no gradient at all."""
    n = len(CASES["gpt2_tiny"]["spec"].lora_shapes())
    have = [f"gpt2_tiny/grad/{i}" in model_golden.files for i in range(n)]
    assert have == [False, False, True, True] * (n // 4)


def test_step_matches_live_reference_at_model_width():
    """Full Gemma-3-1B layer widths (hidden 1152, 4x256 heads, GeGLU 6912, window 512 active) on a
    2-layer stack with a reduced vocabulary, against the reference driver run on this machine."""
    from oracle import model_case
    require_reference()
    from mobilefinetuner_b200 import configs as Cf
    spec = Cf.reduced(Cf.GEMMA3_1B, vocab=4096, layers=2, global_every=2)
    case = dict(spec=spec, batch=1, seq=640, seeds=(401, 402, 403), norm_jitter=0.05)
    from mobilefinetuner_b200 import synth
    params = synth.make_params(spec, 401, 0.05)
    lora = synth.make_lora(spec, 402)
    ids, labels = synth.make_batch(spec, 1, 640, 403)
    ref = model_case.run_reference_step(spec, params, lora, ids, labels, **STEP)
    loss, grads, after, lora0 = run_engine(case)
    worst = check(loss, grads, after, lora0, float(ref["loss"][0]), ref["grads"], ref["lora_after"])
    print("worst gradient cosine", worst)


def test_gradient_accumulation_and_zero_grad():
    """Leaf gradients accumulate across backward calls until zero_grad (core/test_autograd_leaf_accum.cpp)."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200.engine import LoraStepEngine
    case = CASES["qwen_tiny"]
    spec = case["spec"]
    eng = LoraStepEngine(spec, case["batch"], case["seq"])
    eng.set_params(synth.make_params(spec, 1, 0.1))
    eng.set_lora(synth.make_lora(spec, 2))
    ids, labels = synth.make_batch(spec, case["batch"], case["seq"], 3)
    eng.forward_backward(ids, labels)
    g1 = eng.grad_bucket().clone()
    eng.forward_backward(ids, labels)
    g2 = eng.grad_bucket().clone()
    assert float((g2 - 2 * g1).abs().max()) <= 1e-3 * float(g1.abs().max())
    eng.zero_grad()
    assert float(eng.grad_bucket().abs().max()) == 0.0
    eng.close()


def test_replayed_step_graph_matches_direct_launches():
    """From the third call with one batch shape the step engine replays a captured CUDA graph: same gradients, same
    loss, and the launch counter keeps counting the kernels a replay runs."""
    from mobilefinetuner_b200 import _lib as L, synth
    from mobilefinetuner_b200.engine import LoraStepEngine
    case = CASES["gemma_tiny"]
    spec = case["spec"]
    eng = LoraStepEngine(spec, case["batch"], case["seq"])
    eng.set_params(synth.make_params(spec, 1, 0.1))
    eng.set_lora(synth.make_lora(spec, 2))
    ids, labels = synth.make_batch(spec, case["batch"], case["seq"], 3)
    losses, grads, launches = [], [], []
    for _ in range(4):                       # direct, capture, replay, replay
        before = L.call("mft_launch_count")
        loss, _ = eng.forward_backward(ids, labels)
        launches.append(L.call("mft_launch_count") - before)
        losses.append(loss)
        grads.append(eng.grad_bucket().clone())
        eng.zero_grad()
    for k in range(1, 4):
        assert abs(losses[k] - losses[0]) <= 1e-5 * abs(losses[0])
        assert float((grads[k] - grads[0]).abs().max()) <= 1e-4 * float(grads[0].abs().max())
        assert launches[k] >= launches[0] - 8 and launches[k] > 0      # replays are counted (memsets are not kernels)
    eng.close()


def test_data_parallel_shards_add_up_to_the_full_batch():
    """What two data-parallel ranks compute: each runs its own samples with the GLOBAL count of scored tokens as the
    loss denominator; the sum of their LoRA-gradient buckets (the all-reduce) is the full-batch gradient."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200.engine import LoraStepEngine
    case = CASES["qwen_tiny"]
    spec = case["spec"]
    B, S = 2, case["seq"]
    eng = LoraStepEngine(spec, B, S)
    eng.set_params(synth.make_params(spec, 1, 0.1))
    eng.set_lora(synth.make_lora(spec, 2))
    ids, labels = synth.make_batch(spec, B, S, 3)
    labels = labels.copy()
    labels[1, S // 2:] = -100                      # unequal numbers of scored tokens per rank
    loss_full, n_full = eng.forward_backward(ids, labels)
    g_full = eng.grad_bucket().clone()
    eng.zero_grad()
    loss_sum = 0.0
    for r in range(B):
        loss_r, n_r = eng.forward_backward(ids[r:r + 1], labels[r:r + 1], n_valid_global=n_full)
        loss_sum += loss_r * n_r / n_full            # ranks report their local mean; the global mean weights by count
    g_sum = eng.grad_bucket().clone()
    assert abs(loss_sum - loss_full) <= 2e-3 * abs(loss_full)
    assert float((g_sum - g_full).abs().max()) <= 5e-3 * float(g_full.abs().max())
    assert cosine(g_sum.cpu().numpy(), g_full.cpu().numpy()) >= 0.9999
    eng.close()


def test_step_driver_accumulates_clips_and_schedules_like_the_trainers():
    """LoraTrainer.train_step == the trainers' loop body: two micro-batches with the loss scaled by 1/2 accumulate,
    the call that closes the window clips with max/(norm + 1e-6), takes the scheduled learning rate and steps Adam.
    Compared with the same sequence issued by hand through the step engine (itself pinned to the reference)."""
    from mobilefinetuner_b200 import _lib as L, synth
    from mobilefinetuner_b200.engine import LoraStepEngine, LoraTrainer
    from oracle import restate as R
    case = CASES["gemma_tiny"]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    params, lora = synth.make_params(spec, 1, 0.1), synth.make_lora(spec, 2)
    batches = [synth.make_batch(spec, B, S, 10 + k) for k in range(4)]
    sched = dict(learning_rate=3e-4, warmup_ratio=0.5, lr_scheduler="cosine", total_updates=4)

    eng = LoraStepEngine(spec, B, S)
    eng.set_params(params); eng.set_lora(lora)
    tr = LoraTrainer(eng, grad_accum_steps=2, max_grad_norm=0.05, weight_decay=0.01, **sched)
    seen = [tr.train_step(*batches[k]) for k in range(4)]
    assert seen[0] == -1.0 and seen[2] == -1.0 and seen[1] > 0 and seen[3] > 0
    assert tr.global_step == 2
    assert abs(tr.last_lr - R.trainer_lr(2, 3e-4, 0.5, "cosine", 4)) <= 1e-10
    got = eng.get_lora()
    tr.close(); eng.close()

    ref = LoraStepEngine(spec, B, S)
    ref.set_params(params); ref.set_lora(lora)
    losses = []
    for step in (1, 2):
        L.call("mft_model_set_loss_scale", ref._h, 0.5)
        for k in (2 * step - 2, 2 * step - 1):
            losses.append(ref.forward_backward(*batches[k])[0])
        L.call("mft_model_optimizer_step", ref._h, R.trainer_lr(step, 3e-4, 0.5, "cosine", 4), 0.9, 0.999, 1e-8, 0.01, 0.05, 1e-6)
    want = ref.get_lora()
    ref.close()
    assert abs(seen[1] - 0.5 * (losses[0] + losses[1])) <= 1e-5 * abs(seen[1])
    # the second window runs on parameters that went through one Adam step in each arm (see below: not bit-identical)
    assert abs(seen[3] - 0.5 * (losses[2] + losses[3])) <= 1e-4 * abs(seen[3])
    # Two runs of the same step are not bit-identical (f32 atomics in the LoRA-gradient and dK/dV reductions), and
    # Adam's early steps move an element by about lr * sign(g): an element whose tiny gradient changes sign between
    # the runs differs by up to 2 lr per step.  Everything else agrees to rounding.
    lr_max = 3e-4
    for a, b in zip(got, want):
        d = np.abs(a - b)
        assert d.max() <= 2 * 2.1 * lr_max
        assert (d <= 1e-6 + 1e-4 * np.abs(b).max()).mean() >= 0.97


def _accum_run(monkeypatch, graph, probe_between):
    """Three optimizer steps of two micro-batches each on one repeated batch; returns the window losses and the
    final adapters.  `graph` selects CUDA-graph replay of the step, `probe_between` adds an evaluation forward
    between the first two micro-batches (so that the call that gets captured starts with clean panels)."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200.engine import LoraStepEngine, LoraTrainer
    case = CASES["gemma_tiny"]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    monkeypatch.setenv("MFT_STEP_GRAPH", "1" if graph else "0")
    eng = LoraStepEngine(spec, B, S)
    eng.set_params(synth.make_params(spec, 1, 0.1)); eng.set_lora(synth.make_lora(spec, 2))
    ids, labels = synth.make_batch(spec, B, S, 10)
    tr = LoraTrainer(eng, grad_accum_steps=2, max_grad_norm=0.0, learning_rate=5e-3, lr_scheduler="constant", total_updates=3)
    losses = []
    for k in range(6):
        out = tr.train_step(ids, labels)
        if k == 0 and probe_between:
            eng.forward_loss(ids, labels)
        if out >= 0:
            losses.append(out)
    got = eng.get_lora()
    tr.close(); eng.close()
    return losses, got


@pytest.mark.parametrize("probe_between", [False, True])
def test_graph_replay_sees_every_optimizer_step(monkeypatch, probe_between):
    """The bf16 LoRA panels the GEMMs read are re-packed from the f32 masters after every optimizer step whether the
    step runs as a replayed CUDA graph or launch by launch: with gradient accumulation the captured call is a second
    micro-batch (panels already clean), and an evaluation forward before it has the same effect.  Both orders must
    train exactly like the uncaptured schedule; with stale panels the loss would not move after the first window."""
    eager_losses, eager_lora = _accum_run(monkeypatch, False, probe_between)
    graph_losses, graph_lora = _accum_run(monkeypatch, True, probe_between)
    assert len(eager_losses) == len(graph_losses) == 3
    assert eager_losses[2] < eager_losses[1] < eager_losses[0] - 1e-3          # lr 5e-3 on a repeated batch: it learns
    for a, b in zip(graph_losses, eager_losses):
        assert abs(a - b) <= 2e-4 * abs(b), (graph_losses, eager_losses)
    # Adam moves an element by about lr per step whatever the gradient's size, and two runs differ in the last bits
    # (f32 atomics), so an element whose tiny gradient changes sign ends up to 2 lr per step apart: bound the worst
    # case by that and ask the typical element to agree far better.
    lr = 5e-3
    for a, b in zip(graph_lora, eager_lora):
        d = np.abs(a - b)
        assert d.max() <= 3 * 2.1 * lr and np.median(d) <= 0.05 * lr


def test_double_buffered_input_gives_the_same_steps():
    """BatchPipeline (next batch copied on a copy stream during the current step, loss read back one step late)
    against the plain one-call-per-step path: same losses, same scored-token counts, same parameters."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200.engine import BatchPipeline, LoraStepEngine
    case = CASES["gemma_tiny"]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    params, lora = synth.make_params(spec, 1, 0.1), synth.make_lora(spec, 2)
    batches = []
    for k in range(5):
        ids, labels = synth.make_batch(spec, B, S, 40 + k)
        labels = labels.copy(); labels[0, S - 1 - k:] = -100
        batches.append((ids, labels))

    plain = LoraStepEngine(spec, B, S)
    plain.set_params(params); plain.set_lora(lora)
    want = []
    for ids, labels in batches:
        want.append(plain.forward_backward(ids, labels))
        plain.optimizer_step(1e-4, max_grad_norm=1.0)
    want_lora = plain.get_lora()
    plain.close()

    eng = LoraStepEngine(spec, B, S)
    eng.set_params(params); eng.set_lora(lora)
    pipe = BatchPipeline(eng, B, S)
    got = list(pipe.run(batches, after_backward=lambda k: eng.optimizer_step(1e-4, max_grad_norm=1.0)))
    got_lora = eng.get_lora()
    eng.close()
    assert [g[0] for g in got] == list(range(5))
    for (k, loss, nv), (wloss, wnv) in zip(got, want):
        assert nv == wnv and abs(loss - wloss) <= 2e-4 * abs(wloss), (k, loss, wloss)
    # Two runs of five Adam steps are not bit-identical (f32 atomics in the gradient reductions; an element whose tiny
    # gradient changes sign moves the other way by up to 2 lr per step): compare the parameter UPDATES as vectors.
    for a, b, p0 in zip(got_lora, want_lora, lora):
        assert np.abs(a - b).max() <= 5 * 2.1 * 1e-4
        assert cosine(a - p0, b - p0) >= 0.97


@pytest.mark.parametrize("name,storage", [("gemma_tiny", "BF16"), ("qwen_tiny", "F32"), ("gpt2_tiny", "F16")])
def test_checkpoint_ingest_and_adapter_files_round_trip(name, storage, tmp_path):
    """A HuggingFace-style checkpoint (HF keys, Linear weights [out,in], F32 / F16 / BF16 storage, two shards + index)
    loaded through mft_model_load_safetensors gives the same model as installing the tensors one by one; an adapter
    saved with mft_model_save_lora_safetensors loads back bit-identically and carries the PEFT-style keys."""
    import ctypes as C
    import json
    import struct
    import torch
    from mobilefinetuner_b200 import _lib as L, synth
    from mobilefinetuner_b200.engine import LoraStepEngine
    from test_safetensors_cpu import bf16_bits, write_container
    case = CASES[name]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    params, lora = synth.make_params(spec, 1, 0.1), synth.make_lora(spec, 2)
    if storage == "F16":                                 # what the file can hold
        params = [p.astype(np.float16).astype(np.float32) for p in params]
    elif storage == "BF16":
        params = [(bf16_bits(p).astype(np.uint32) << 16).view(np.float32).reshape(p.shape) for p in params]
    ids, labels = synth.make_batch(spec, B, S, 3)
    ref = LoraStepEngine(spec, B, S)
    ref.set_params(params); ref.set_lora(lora)
    want_loss = ref.forward_loss(ids, labels)

    def store(a):
        if storage == "F32":
            return "F32", a.astype(np.float32)
        if storage == "F16":
            return "F16", a.astype(np.float16)
        return "BF16", bf16_bits(a)

    tensors = {}
    for i, p in enumerate(params):
        key, tr = C.create_string_buffer(256), C.c_int32()
        L.call("mft_model_hf_key", ref._h, i, key, 256, C.byref(tr))
        if key.value:
            tensors[key.value.decode()] = store(p.T if tr.value else p)
    assert any(k.endswith("q_proj.weight") or k.endswith("c_attn.weight") for k in tensors)
    d = tmp_path / "ckpt"
    d.mkdir()
    items = list(tensors.items())
    half = len(items) // 2
    write_container(d / "model-00001-of-00002.safetensors", dict(items[:half]), {"format": "pt"})
    write_container(d / "model-00002-of-00002.safetensors", dict(items[half:]))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors") for i, (k, _) in enumerate(items)}}))

    eng = LoraStepEngine(spec, B, S)
    L.call("mft_model_load_safetensors", eng._h, str(d).encode())
    eng.set_lora(lora)
    got_loss = eng.forward_loss(ids, labels)
    assert abs(got_loss - want_loss) <= 1e-6 * abs(want_loss)

    # adapter save -> load into a fresh engine
    path = tmp_path / "adapter.safetensors"
    L.call("mft_model_save_lora_safetensors", ref._h, str(path).encode())
    raw = path.read_bytes()
    header = json.loads(raw[8:8 + struct.unpack("<Q", raw[:8])[0]])
    assert header["__metadata__"]["rank"] == str(spec.lora_rank) and "targets" in header["__metadata__"]
    keys = [k for k in header if k != "__metadata__"]
    assert keys == sorted(keys) and all(k.startswith("layer.") and k.rsplit(".", 1)[1] in ("lora_A", "lora_B") for k in keys)
    assert len(keys) == len(lora)
    other = LoraStepEngine(spec, B, S)
    other.set_params(params)
    L.call("mft_model_load_lora_safetensors", other._h, str(path).encode())
    for a, b in zip(other.get_lora(), ref.get_lora()):
        np.testing.assert_array_equal(a, b)
    assert abs(other.forward_loss(ids, labels) - want_loss) <= 1e-6 * abs(want_loss)
    ref.close(); eng.close(); other.close()


def test_evaluation_drivers_perplexity_and_letter_scores():
    """eval_ppl aggregation over batches and MMLU-style letter scoring (log_softmax of the last position read at the
    candidate ids), against the restated aggregation and a float64 projection of the engine's own final hidden state."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200.engine import LoraStepEngine
    from oracle import restate as R
    case = CASES["qwen_tiny"]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    params = synth.make_params(spec, 1, 0.1)
    eng = LoraStepEngine(spec, B, S)
    eng.set_params(params); eng.set_lora(synth.make_lora(spec, 2))
    batches = []
    for k in range(3):
        ids, labels = synth.make_batch(spec, B, S, 20 + k)
        labels = labels.copy(); labels[0, : 3 + k] = -100
        batches.append((ids, labels))
    nll, ppl, tokens = eng.perplexity(batches)
    losses = [eng.forward_loss(i, l) for i, l in batches]
    w_nll, w_ppl, w_tokens = R.ppl_accumulate(losses, [l for _, l in batches])
    assert tokens == w_tokens and abs(nll - w_nll) <= 1e-6 * w_nll and abs(ppl - w_ppl) <= 1e-5 * w_ppl

    prompt = batches[0][0][0, : S - 3]
    cand = np.array([5, 17, spec.vocab - 1, 0, spec.vocab + 3], np.int32)     # the last id is outside the vocabulary
    got = eng.score_tokens(prompt, cand)
    hidden = eng.final_hidden(prompt.size)[-1].astype(np.float64)              # final-norm output of the last position (bf16 values)
    import torch
    table = torch.from_numpy(params[0]).bfloat16().double().numpy()           # the tied table as the GPU holds it
    logits = table @ hidden
    logp = logits - (np.log(np.exp(logits - logits.max()).sum()) + logits.max())
    assert got[4] == np.float32(-1e30)
    np.testing.assert_allclose(got[:4], logp[cand[:4]], rtol=0, atol=2e-3)
    eng.close()


@pytest.mark.parametrize("name", ["gemma_tiny", "qwen_tiny", "gpt2_tiny"])
def test_merge_to_base_and_unmerge(name):
    """LoRALinear::merge_to_base / unmerge_from_base on the device weights: the merged forward agrees with the
    adapter forward (bf16 path tolerance), equals an engine that was GIVEN W + scale * A B (the reference's update
    rule evaluated in numpy: double accumulation, float update, rounded to the bf16 storage) with idle adapters, training
    is refused while merged, and unmerge brings the original loss back."""
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200._lib import MftError
    from mobilefinetuner_b200.configs import GEMMA
    from mobilefinetuner_b200.engine import LoraStepEngine
    case = CASES[name]
    spec = case["spec"]
    B, S = case["batch"], case["seq"]
    params = [synth.bf16_round(p) if p.ndim == 2 else p for p in synth.make_params(spec, case["seeds"][0], case["norm_jitter"])]
    lora = synth.make_lora(spec, case["seeds"][1])
    ids, labels = synth.make_batch(spec, B, S, case["seeds"][2])
    eng = LoraStepEngine(spec, B, S)
    eng.set_params(params); eng.set_lora(lora)
    loss0 = eng.forward_loss(ids, labels)
    eng.merge_to_base()
    assert eng.is_merged
    loss_m = eng.forward_loss(ids, labels)
    assert abs(loss_m - loss0) <= LOSS_REL * abs(loss0)
    with pytest.raises(MftError):
        eng.forward_backward(ids, labels)
    with pytest.raises(MftError):
        eng.set_lora(lora)
    eng.merge_to_base()                                   # a second merge is a no-op, as in the reference
    assert abs(eng.forward_loss(ids, labels) - loss_m) <= 1e-6 * abs(loss_m)

    # the same update in numpy, applied to the frozen weights of a second engine whose adapters contribute nothing
    linear_idx = [i for i, (kind, _) in enumerate(spec.param_shapes()) if kind == "linear"]
    per_layer = len(linear_idx) // spec.layers
    order = {"q_proj": 0, "k_proj": 1, "v_proj": 2, "o_proj": 3, "gate_proj": 4, "up_proj": 5, "down_proj": 6,
             "c_attn": 0, "c_proj": 1, "c_fc": 2, "mlp_c_proj": 3}
    names = [n for n, _ in spec.lora_shapes()]
    per_layer_lora = len(names) // spec.layers
    scale = np.float32(spec.lora_alpha / spec.lora_rank)
    merged = [p.copy() for p in params]
    for j in range(0, len(names), 2):
        layer, target = j // per_layer_lora, names[j][:-2]
        A, Bm = lora[j].astype(np.float64), lora[j + 1].astype(np.float64)
        delta = (A.T @ Bm.T) if spec.family == GEMMA else (A @ Bm)               # [in, out]
        w = merged[linear_idx[layer * per_layer + order[target]]]
        w += scale * delta.astype(np.float32)
    idle = [a if n.endswith(".A") else np.zeros_like(a) for a, (n, _) in zip(lora, spec.lora_shapes())]
    eng2 = LoraStepEngine(spec, B, S)
    eng2.set_params(merged); eng2.set_lora(idle)
    loss2 = eng2.forward_loss(ids, labels)
    eng2.close()
    assert abs(loss2 - loss_m) <= 1e-6 * abs(loss_m)

    eng.unmerge_from_base()
    assert not eng.is_merged
    assert abs(eng.forward_loss(ids, labels) - loss0) <= 1e-6 * abs(loss0)
    loss_t, _ = eng.forward_backward(ids, labels)         # training works again
    assert abs(loss_t - loss0) <= LOSS_REL * abs(loss0)
    eng.close()


def test_out_of_range_token_raises():
    from mobilefinetuner_b200 import synth
    from mobilefinetuner_b200._lib import MftError
    from mobilefinetuner_b200.engine import LoraStepEngine
    case = CASES["qwen_tiny"]
    spec = case["spec"]
    eng = LoraStepEngine(spec, case["batch"], case["seq"])
    eng.set_params(synth.make_params(spec, 1))
    eng.set_lora(synth.make_lora(spec, 2))
    ids, labels = synth.make_batch(spec, case["batch"], case["seq"], 3)
    ids[0, 3] = spec.vocab
    with pytest.raises(MftError):
        eng.forward_backward(ids, labels)
    eng.close()
