"""Compile the C-ABI CUDA library in-tree for sm_100a, and the torch-extension
shim of the decode operator on top of it.

``python -m mac_attention_b200.build`` writes ``mac_attention_b200/libmac_b200.so``
and ``mac_attention_b200/mac_b200_torch.so`` next to this file.  nvcc
cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmac_b200.so"
SOURCES = ["mac_b200_api.cu", "mac_b200_prefill.cu", "mac_b200_decode.cu", "mac_b200_rope.cu",
           "mac_b200_downdate.cu", "mac_b200_prefill_build.cu", "mac_b200_prefill_sink_tc.cu"]
HEADERS = [CSRC / "mac_b200_common.h", CSRC / "mac_b200_state_math.cuh",
           PKG.parent / "include" / "mac_b200.h"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build libmac_b200.so")
    return cand


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + HEADERS
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "-Xptxas", "-v" if verbose else "-warn-spills",
        "-diag-suppress", "177",
        "-shared", "-Xcompiler", "-fPIC",
        "-o", str(LIB),
        *[str(CSRC / s) for s in SOURCES],
    ]
    extra = os.environ.get("MAC_B200_NVCC_FLAGS", "").split()
    cmd[1:1] = extra
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return LIB


SHIM = PKG / "mac_b200_torch.so"
SHIM_SRC = CSRC / "mac_b200_torch.cpp"


def shim_is_stale() -> bool:
    if not SHIM.exists():
        return True
    t = SHIM.stat().st_mtime
    return any(d.stat().st_mtime > t for d in (SHIM_SRC, PKG.parent / "include" / "mac_b200.h"))


def build_shim(force: bool = False, verbose: bool = False) -> Path:
    """The pybind module that takes ``torch.Tensor`` arguments and calls the C ABI:
    one C++ file against the torch headers, linked to ``libmac_b200.so`` next to it."""
    if not force and not shim_is_stale():
        return SHIM
    build()
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cuda_home = Path(_nvcc()).resolve().parents[1]
    incs = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(cuda_home / "include")]
    libdirs = cpp_extension.library_paths()
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=mac_b200_torch",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-attributes",
           *[f"-I{i}" for i in incs], str(SHIM_SRC), "-o", str(SHIM),
           *[f"-L{d}" for d in libdirs], f"-L{PKG}",
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-l:libmac_b200.so",
           "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in libdirs]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"{cxx} failed with exit code {res.returncode} building the torch shim")
    return SHIM


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_shim(force="--force" in sys.argv, verbose="-v" in sys.argv))
