"""Test infrastructure: runs the compiled, unmodified reference (oracle/_ref/ref_driver_*)
on a case directory and reads its results back.

Only tests/, the smoke check and bench.py's CPU-baseline leg may import this
module; the product never does.  The driver binaries are built by
`make -C oracle` (see oracle/Makefile) from the reference's own sources.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
REF_DIR = ORACLE_DIR / "_ref"


def _works(binary: Path) -> bool:
    try:
        r = subprocess.run([str(binary)], capture_output=True, timeout=20)
        return r.returncode == 2 and b"usage" in r.stderr
    except Exception:
        return False


_cached: dict[str, Path | None] = {}


def driver(prefer_blas: bool = True) -> Path | None:
    """Path of a working reference driver, or None when oracle/_ref was not built."""
    key = "blas" if prefer_blas else "noblas"
    if key in _cached:
        return _cached[key]
    order = ["ref_driver_blas", "ref_driver_noblas"] if prefer_blas else ["ref_driver_noblas", "ref_driver_blas"]
    found = None
    for name in order:
        p = REF_DIR / name
        if p.exists() and _works(p):
            found = p
            break
    _cached[key] = found
    return found


def kind(binary: Path) -> str:
    return "blas" if binary.name.endswith("_blas") else "noblas"


def write_case(case_dir: Path, params: dict, tensors: dict[str, np.ndarray]) -> None:
    case_dir.mkdir(parents=True, exist_ok=True)
    with open(case_dir / "case.txt", "w") as f:
        for k, v in params.items():
            f.write(f"{k} {v}\n")
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        if arr.dtype not in (np.float32, np.int32):
            raise TypeError(f"{name}: reference tensors are float32 or int32, got {arr.dtype}")
        path = case_dir / f"{name}.npy"
        path.parent.mkdir(parents=True, exist_ok=True)
        np.save(path, arr)


def read_outputs(case_dir: Path) -> dict[str, np.ndarray]:
    out = {}
    for p in sorted((case_dir / "out").glob("*.npy")):
        out[p.stem] = np.load(p)
    timing = case_dir / "out" / "timing.txt"
    if timing.exists():
        out["_timing"] = timing.read_text()
    return out


def run(mode: str, params: dict, tensors: dict[str, np.ndarray], *, extra_files: dict[str, str] | None = None,
        threads: int | None = None, prefer_blas: bool = True, keep: Path | None = None, timeout: float = 3600) -> dict:
    """Run `ref_driver <mode>` on a fresh case directory and return its outputs."""
    binary = driver(prefer_blas)
    if binary is None:
        raise FileNotFoundError("oracle/_ref has no working ref_driver: run `make -C oracle` where the reference is mounted")
    tmp = Path(keep) if keep else Path(tempfile.mkdtemp(prefix="mft_oracle_"))
    try:
        write_case(tmp, params, tensors)
        for name, content in (extra_files or {}).items():
            (tmp / name).write_text(content)
        env = dict(os.environ)
        if threads:
            env["ORACLE_BLAS_THREADS"] = str(threads)
            env["OPENBLAS_NUM_THREADS"] = str(threads)
        r = subprocess.run([str(binary), mode, str(tmp)], capture_output=True, text=True, env=env, timeout=timeout)
        if r.returncode != 0:
            raise RuntimeError(f"ref_driver {mode} failed ({r.returncode}): {r.stderr[-2000:]}")
        out = read_outputs(tmp)
        out["_driver"] = kind(binary)
        return out
    finally:
        if not keep:
            shutil.rmtree(tmp, ignore_errors=True)


def run_op(op: str, tensors: dict[str, np.ndarray], **params) -> dict:
    p = {"op": op}
    p.update(params)
    return run("op", p, tensors)
