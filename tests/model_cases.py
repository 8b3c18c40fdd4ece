"""Reduced whole-model parity cases shared by the golden generator and the GPU tests:
full architecture features (GQA, sliding + global layers, QK-norm, tied head, biases, odd
vocabulary), small enough for the CPU reference to finish in seconds."""
from mobilefinetuner_b200 import configs as Cf

CASES = {
    "gemma_tiny": dict(spec=Cf.reduced(Cf.GEMMA3_1B, vocab=2048, hidden=256, inter=512, layers=3, n_heads=4, n_kv_heads=1,
                                       head_dim=256, sliding_window=16, global_every=3, lora_rank=16, lora_alpha=32.0),
                       batch=2, seq=40, seeds=(101, 102, 103), norm_jitter=0.1),
    "gemma_r8_hd64": dict(spec=Cf.reduced(Cf.GEMMA3_270M, vocab=1000, hidden=128, inter=256, layers=2, n_heads=4, n_kv_heads=2,
                                          head_dim=64, sliding_window=8, global_every=2, query_pre_attn_scalar=64.0),
                          batch=3, seq=24, seeds=(111, 112, 113), norm_jitter=0.1),
    "qwen_tiny": dict(spec=Cf.reduced(Cf.QWEN25_05B, vocab=3000, hidden=256, inter=512, layers=2, n_heads=4, n_kv_heads=2, head_dim=64),
                      batch=2, seq=48, seeds=(201, 202, 203), norm_jitter=0.1),
    "gpt2_tiny": dict(spec=Cf.reduced(Cf.GPT2_SMALL, vocab=1001, hidden=128, inter=512, layers=2, n_heads=2, n_kv_heads=2,
                                      head_dim=64, n_positions=64),
                      batch=2, seq=32, seeds=(301, 302, 303), norm_jitter=0.1),
}
STEP = dict(lr=2e-4, max_grad_norm=1.0)
