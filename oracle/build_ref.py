"""Build the reference's own CUDA kernels for sm_100a into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or
anything it produces; only ``tests/``, ``bench.py`` (baseline legs) and
``__graft_entry__.build()`` may use it.

The reference ships its decode kernel (``mac_decode_persistent.cu``) and its
prefill ring-update kernels (``mac_prefill_update_cache.cu``) as single-file
PyTorch extensions whose own loader (``integrations/sglang/bridge.py:172-269``)
only emits sm_90/sm_90a SASS.  Both files compile unmodified for sm_100a, so
this recipe compiles them *from where they lie* in the read-only reference
checkout (no source is copied into this repository) with the reference's other
flags kept (``-dlcm=cg``, the ``-U__CUDA_NO_*`` switches, ``--use_fast_math``
as in the published benchmark runs).  The resulting ``.so`` files are used

* as a device-side oracle for hit/match decisions (same inputs, compare the
  decision arrays bit for bit), and
* as a same-box timed baseline next to FlashInfer.

The build needs the reference checkout, so it only runs where that exists;
elsewhere the prebuilt ``oracle/_ref/*.so`` files are loaded if present.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REF_ROOT = Path(os.environ.get("MAC_REFERENCE_ROOT", "/root/reference"))
CSRC = REF_ROOT / "attention/src/mac_attention/integrations/sglang/csrc"

DECODE_NAME = "mac_ref_persistent_decode_sm100a"
PREFILL_NAME = "mac_ref_prefill_update_cache_sm100a"
ROPE_NAME = "mac_ref_decode_rope_preserve_sm100a"
DOWNDATE_NAME = "mac_ref_merge_downdate_cache_sm100a"

_ARCH = ["-gencode=arch=compute_100a,code=sm_100a"]


def _load(name: str, source: Path, cuda_flags: list[str], verbose: bool):
    from torch.utils import cpp_extension

    build_dir = OUT / name
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return cpp_extension.load(
        name=name,
        sources=[str(source)],
        extra_cuda_cflags=cuda_flags,
        extra_cflags=["-O3", "-std=c++17"],
        build_directory=str(build_dir),
        verbose=verbose,
    )


def build_decode(verbose: bool = False):
    flags = [
        "-O3", "-std=c++17",
        "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        *_ARCH, "-Xptxas", "-dlcm=cg", "--use_fast_math",
    ]
    return _load(DECODE_NAME, CSRC / "mac_decode_persistent.cu", flags, verbose)


def build_prefill(verbose: bool = False):
    flags = [
        "-O3", "--use_fast_math", "-std=c++17",
        "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", *_ARCH, "-Xptxas", "-dlcm=cg",
    ]
    return _load(PREFILL_NAME, CSRC / "mac_prefill_update_cache.cu", flags, verbose)


def build_rope(verbose: bool = False):
    flags = ["-O3", "-std=c++17", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", *_ARCH]
    return _load(ROPE_NAME, CSRC / "mac_decode_rope_preserve.cu", flags, verbose)


def build_downdate(verbose: bool = False):
    flags = ["-O3", "--use_fast_math", "-Xptxas", "-O3", "-Xptxas", "-dlcm=ca", *_ARCH,
             "-DTILE_D=1024", "-DTHREADS=256"]
    return _load(DOWNDATE_NAME, CSRC / "mac_merge_downdate_cache.cu", flags, verbose)


# --------------------------------------------------------------------------- the reference's own tests
SUITE = OUT / "ref_suite"
_SUITE_FILES = {
    # reference file (relative to its project root) -> place in the staged suite
    "attention/src/mac_attention/integrations/sglang/bridge.py":
        "pkg/mac_attention/integrations/sglang/bridge.py",
    "attention/tests/test_mac_persistent_decode.py": "tests/test_mac_persistent_decode.py",
    "attention/tools/check_mac_persistent_decode.py": "tools/check_mac_persistent_decode.py",
    "attention/tools/check_front_sink_recurrence.py": "tools/check_front_sink_recurrence.py",
}


def stage_reference_suite() -> Path | None:
    """Stage the reference's own kernel tests, its checker tools and its loader
    module -- unmodified, byte for byte -- under ``oracle/_ref/ref_suite`` (kept
    out of the history like everything else in ``oracle/_ref``), so that
    ``tests/test_reference_suite_gpu.py`` can run them against this library on a
    box where the reference checkout is not mounted.  The package ``__init__``
    files around the loader are empty files of our own (the reference's import
    its SGLang hooks, which need SGLang)."""
    import shutil

    if not REF_ROOT.exists():
        return SUITE if SUITE.exists() else None
    for src, dst in _SUITE_FILES.items():
        if not (REF_ROOT / src).exists():
            continue
        target = SUITE / dst
        target.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(REF_ROOT / src, target)
    for pkg in ("pkg/mac_attention", "pkg/mac_attention/integrations",
                "pkg/mac_attention/integrations/sglang"):
        (SUITE / pkg).mkdir(parents=True, exist_ok=True)
        (SUITE / pkg / "__init__.py").write_text("")
    return SUITE


def _import_prebuilt(name: str):
    """Import ``oracle/_ref/<name>/<name>.so`` without rebuilding."""
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    so = OUT / name / f"{name}.so"
    if not so.exists():
        return None
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_decode():
    """Prebuilt reference decode extension, or ``None`` when it was never built."""
    return _import_prebuilt(DECODE_NAME)


def load_prefill():
    return _import_prebuilt(PREFILL_NAME)


def load_rope():
    return _import_prebuilt(ROPE_NAME)


def load_downdate():
    return _import_prebuilt(DOWNDATE_NAME)


def main() -> int:
    if not CSRC.exists():
        print(f"reference sources not found under {CSRC}; nothing built")
        return 0
    which = sys.argv[1:] or ["prefill", "rope", "downdate", "decode"]
    if "prefill" in which:
        build_prefill(verbose=True)
    if "rope" in which:
        build_rope(verbose=True)
    if "downdate" in which:
        build_downdate(verbose=True)
    if "decode" in which:
        build_decode(verbose=True)
    stage_reference_suite()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
