"""Compile the C-ABI CUDA library in-tree for sm_100a.

``python -m mac_attention_b200.build`` writes ``mac_attention_b200/libmac_b200.so``
next to this file.  nvcc cross-compiles without a GPU.
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
           "mac_b200_downdate.cu", "mac_b200_prefill_build.cu"]
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


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
