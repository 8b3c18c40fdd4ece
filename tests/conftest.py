import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


class Golden:
    """Accessor for tests/golden/ops_golden.npz (inputs and outputs of the compiled reference)."""

    def __init__(self):
        self._z = np.load(ROOT / "tests" / "golden" / "ops_golden.npz")

    def case(self, name):
        ins, outs, params = {}, {}, {}
        for key in self._z.files:
            if key.startswith(name + "/"):
                _, kind, leaf = key.split("/", 2)
                {"in": ins, "out": outs, "param": params}[kind][leaf] = self._z[key]
        if not ins:
            raise KeyError(name)
        return ins, outs, {k: v.item() for k, v in params.items()}


@pytest.fixture(scope="session")
def golden():
    return Golden()


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def cosine(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-300))
