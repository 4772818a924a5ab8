"""In-tree build of the native libraries (nvcc for sm_100a, g++ for host code).

Each ``csrc/<name>.cu`` becomes ``_lib/libftb_<name>.so`` and each ``csrc/<name>.cpp`` becomes
``_lib/libftb_<name>.so``; they are loaded with ``ctypes`` (see ``flextrain_b200/ops/cuda.py``),
so a build takes seconds per file and needs neither a GPU nor PyTorch headers.

    python -m flextrain_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_HOME = Path(NVCC).resolve().parent.parent

CUDA_SOURCES = ["gemm_tcgen05", "elementwise", "attention", "comm", "moe", "noalloc", "gdn", "seqmix"]
CPP_SOURCES = ["dp_solver", "copy_engine"]
PYEXT_SOURCES = ["fastcall"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]


def _newer(src: Path, out: Path, extra=()) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(p.exists() and p.stat().st_mtime > t for p in (src, *extra))


def lib_path(name: str) -> Path:
    return LIB / f"libftb_{name}.so"


def build_all(force: bool = False, verbose: bool = False) -> dict:
    """Compile every native source that exists. Returns ``{name: path}``; raises on a compile error."""
    LIB.mkdir(exist_ok=True)
    built = {}
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    for name in CUDA_SOURCES:
        src = CSRC / f"{name}.cu"
        if not src.exists():
            continue
        out = lib_path(name)
        if force or _newer(src, out, headers):
            cmd = [NVCC, *NVCC_FLAGS, "-I", str(CSRC), "-o", str(out), str(src), "-lcudart"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            (LIB / f"{name}.ptxas.log").write_text(r.stderr)
            if verbose:
                print(r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr[-4000:]}")
        built[name] = out
    for name in CPP_SOURCES:
        src = CSRC / f"{name}.cpp"
        if not src.exists():
            continue
        out = lib_path(name)
        if force or _newer(src, out, headers):
            cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", "-I", str(CUDA_HOME / "include"),
                   "-I", str(CSRC), "-o", str(out), str(src)]
            if name == "copy_engine":
                cmd += ["-L", str(CUDA_HOME / "lib64"), "-lcudart", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {src}:\n{r.stderr[-4000:]}")
        built[name] = out
    for name in PYEXT_SOURCES:
        src = CSRC / f"{name}.cpp"
        if not src.exists():
            continue
        suffix = sysconfig.get_config_var("EXT_SUFFIX")
        out = LIB / f"_ftb_{name}{suffix}"
        if force or _newer(src, out, headers):
            cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-I", sysconfig.get_paths()["include"],
                   "-I", str(CUDA_HOME / "include"), "-o", str(out), str(src)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {src}:\n{r.stderr[-4000:]}")
        built[name] = out
    return built


if __name__ == "__main__":
    out = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for k, v in out.items():
        print(f"{k}: {v}")
