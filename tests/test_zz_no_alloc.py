"""GPU test of mft_attn_bwd_noalloc, the attention backward for hosts that cannot allocate device
memory where they call it (its row-sum scratch is a fixed array inside the library).  Called through
the C ABI twice in a row - the second time on a different, smaller problem, so stale scratch contents
from the first call would show - and compared with mft_attn_bwd, which takes the scratch from the
caller.  Both entry points run the same kernels, so the results must be identical.  Collected last on
purpose: a run that stops at the first failure has then already run every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, b, nh, nkv, s, hd):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(b, s, h, hd, device="cuda", generator=g).bfloat16().permute(0, 2, 1, 3)
    return mk(nh), mk(nkv), mk(nkv), mk(nh)


def test_noalloc_backward_matches_regular_entry_point_twice():
    from mobilefinetuner_b200 import ops as O
    # the last two shapes (head_dim 256, sequence a multiple of 128) take the tensor-memory dQ kernel, which reads the
    # row sums straight from the built-in array; the first two take the mma.sync kernels
    for seed, shape, window in [(1, (2, 4, 1, 300, 256), 64), (2, (1, 6, 2, 129, 64), 0), (3, (1, 4, 1, 256, 256), 0), (4, (1, 4, 1, 256, 256), 64)]:
        q, k, v, d_o = _problem(seed, *shape)
        scale = shape[-1] ** -0.5
        o, lse = O.attention_fwd(q, k, v, scale, window)
        want = O.attention_bwd(q, k, v, o, d_o, lse, scale, window, split_heads=False)   # the same kernels: bit-identical
        got = O.attention_bwd_noalloc(q, k, v, o, d_o, lse, scale, window)
        torch.cuda.synchronize()
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            assert torch.isfinite(a.float()).all(), name
            assert torch.equal(a, b), f"{name}: max diff {float((a.float() - b.float()).abs().max())}"


def test_noalloc_rejects_problems_beyond_its_scratch():
    from mobilefinetuner_b200 import ops as O
    from mobilefinetuner_b200._lib import MftError
    b, nh, s, hd = 1, 1, (1 << 20) + 64, 64          # batch*heads*seq just over the 2**20-row limit
    q = torch.zeros(b, s, nh, hd, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    lse = torch.zeros(b, nh, s, device="cuda")
    with pytest.raises(MftError, match="exceeds the built-in scratch"):
        O.attention_bwd_noalloc(q, q, q, q, q, lse, 0.125, 0)
