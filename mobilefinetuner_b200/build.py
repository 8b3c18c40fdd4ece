"""Builds libmft_cuda.so (all CUDA kernels + the C ABI + the C++ step engine) in-tree.

nvcc cross-compiles for sm_100a without a GPU, so this runs on a CPU-only
machine; the resulting shared object sits next to the sources and is what the
ctypes binding loads.

    python -m mobilefinetuner_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libmft_cuda.so"
OPERATORS = PKG / "operator"
OPERATORS_LIB = PKG / "libmft_operators.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))):
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    stamp = OBJ / (src.stem + ".sha")
    dig = _digest(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dig)
    (OBJ / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    return obj, res.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source under csrc/ for sm_100a and link libmft_cuda.so."""
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ.glob("*.sha"):
            f.unlink()
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [str(o) for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    newest = max(Path(o).stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *objs, "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    build_operators(force)
    build_cpp_tests()
    return LIB


def build_operators(force: bool = False) -> Path:
    """Compile the C++ operator API (namespace ops: Tensor, autograd, ops::, LoRALinear, Adam) that sits on
    top of the C ABI into libmft_operators.so."""
    # the two dataset-driven trainer classes need the reference's dataset / tokenizer host code: they are built by
    # operator/CMakeLists.txt when that code is available, not here
    srcs = sorted(p for p in OPERATORS.glob("finetune_ops/*/*.cpp") if p.name not in ("trainer.cpp", "gemma_trainer.cpp"))
    hdrs = sorted(OPERATORS.glob("finetune_ops/*/*.h")) + sorted((PKG.parent / "include").glob("*.h"))
    newest = max(p.stat().st_mtime for p in srcs + hdrs + [LIB])
    if not force and OPERATORS_LIB.exists() and OPERATORS_LIB.stat().st_mtime >= newest:
        return OPERATORS_LIB
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", f"-I{OPERATORS}", f"-I{OPERATORS / 'finetune_ops'}", f"-I{OPERATORS / 'include'}",
           f"-I{PKG.parent / 'include'}", *map(str, srcs), f"-L{PKG}", "-lmft_cuda", "-Wl,-rpath,$ORIGIN", "-o", str(OPERATORS_LIB)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building libmft_operators.so failed:\n{res.stdout}\n{res.stderr}")
    return OPERATORS_LIB


def build_cpp_tests(name: str = "auto_trainer_step") -> Path:
    """Compile tests/cpp/<name>.cpp against the C++ API (auto_trainer_step: driven like the reference's own
    AutoTrainer test; safetensors_reader: the checkpoint reader classes)."""
    src = PKG.parent / "tests" / "cpp" / f"{name}.cpp"
    exe = OBJ / name
    if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, OPERATORS_LIB.stat().st_mtime):
        return exe
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-std=c++17", "-O1", f"-I{OPERATORS}", f"-I{OPERATORS / 'finetune_ops'}", f"-I{OPERATORS / 'include'}", f"-I{PKG.parent / 'include'}", str(src),
           f"-L{PKG}", "-lmft_operators", "-lmft_cuda", f"-Wl,-rpath,{PKG}", "-Wl,-rpath,$ORIGIN/../..", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {name} failed:\n{res.stdout}\n{res.stderr}")
    return exe


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
