"""Parity criteria shared by the whole-model GPU tests: loss relative error <= 2e-3, per-tensor LoRA-gradient
cosine >= 0.999, and after one optimizer step |p' - p'_ref| <= 2e-2 * max(|p'_ref|, lr) on >= 97 % of the elements."""
import numpy as np

from conftest import cosine
from model_cases import STEP

LOSS_REL, GRAD_COS, STEP_REL = 2e-3, 0.999, 2e-2


def check(loss, grads, after, lora0, ref_loss, ref_grads, ref_after):
    assert abs(loss - ref_loss) <= LOSS_REL * abs(ref_loss), (loss, ref_loss)
    worst = 1.0
    stats = []
    for i, (g, rg) in enumerate(zip(grads, ref_grads)):
        if rg is None:
            assert g is None, f"tensor {i}: the reference delivers no gradient here"
            assert np.array_equal(after[i], lora0[i]), f"tensor {i} must not move"
            continue
        c = cosine(g, rg)
        worst = min(worst, c)
        assert c >= GRAD_COS, f"tensor {i}: gradient cosine {c}"
        rel_l2 = float(np.linalg.norm(g - rg) / np.linalg.norm(rg))
        stats.append((i, c, rel_l2))
    print("gradient (tensor, cosine, relL2):", " ".join(f"{i}:{c:.5f}/{r:.3f}" for i, c, r in stats))
    lr = STEP["lr"]
    fracs = []
    for i, (a, ra) in enumerate(zip(after, ref_after)):
        tol = STEP_REL * np.maximum(np.abs(ra), lr)
        # Adam's first step is +-lr*sign(g): elements whose tiny gradient flips sign under bf16 move 2*lr
        frac = float((np.abs(a - ra) <= tol).mean())
        fracs.append(frac)
        assert frac >= 0.97, f"tensor {i}: only {frac:.4f} of updated parameters within tolerance"
        assert np.abs(a - ra).max() <= 2.5 * lr
    print("fraction of updated parameters within 2e-2:", " ".join(f"{f:.4f}" for f in fracs))
    return worst
