"""Drop-in replacement for the reference's extension loader.

The reference obtains its kernels only through
``mac_attention.integrations.sglang.bridge.load_mac_persistent_decode_extension``
and ``load_mac_prefill_update_cache_extension`` (bridge.py:172-187, 211-269 in
the reference project); the returned module objects only need attributes with
the operator names.  The loaders here return such objects backed by the sm_100a
library, and :func:`install` swaps them into the reference's ``bridge`` module
(and into hook modules that already bound the names at import) so the
reference's hooks, tests and tools run unchanged.
"""
from __future__ import annotations

import sys
from functools import lru_cache
from types import SimpleNamespace
from typing import Any

from . import _abi


@lru_cache(maxsize=4)
def load_mac_persistent_decode_extension(verbose: bool = False, fast_math: bool | None = None) -> Any:
    """Same call as the reference loader; ``fast_math`` is accepted and has no effect
    (the kernel always uses the approximate exp2/log2 units, as the reference's
    production build does)."""
    _abi.load_library()
    from . import ops

    return SimpleNamespace(
        mac_persistent_decode_bf16=ops.mac_persistent_decode_bf16,
        mac_persistent_decode_bf16_noalloc=ops.mac_persistent_decode_bf16_noalloc,
        mac_persistent_decode_bf16_lean=ops.mac_persistent_decode_bf16_lean,
        query_status=ops.query_status,
        launch_info=ops.launch_info,
    )


@lru_cache(maxsize=1)
def load_mac_prefill_update_cache_extension(verbose: bool = False) -> Any:
    _abi.load_library()
    from . import ops

    return SimpleNamespace(
        mac_prefill_update_cache=ops.mac_prefill_update_cache,
        mac_mark_persistent_ready=ops.mac_mark_persistent_ready,
        mac_invalidate_persistent_ready=ops.mac_invalidate_persistent_ready,
        mac_update_request_state=ops.mac_update_request_state,
        # not in the reference module: downdate + ring write + ready mark in one pass
        mac_prefill_downdate_update_cache=ops.mac_prefill_downdate_update_cache,
    )


@lru_cache(maxsize=1)
def load_mac_decode_rope_preserve_extension(verbose: bool = False) -> Any:
    _abi.load_library()
    from . import ops

    return SimpleNamespace(mac_decode_rope_preserve_q_bf16=ops.mac_decode_rope_preserve_q_bf16)


@lru_cache(maxsize=1)
def load_mac_merge_downdate_cache_extension(verbose: bool = False) -> Any:
    _abi.load_library()
    from . import ops

    return SimpleNamespace(
        mac_update_then_downdate_bf16_inplace=ops.mac_update_then_downdate_bf16_inplace)


_PATCHED = ("load_mac_persistent_decode_extension", "load_mac_prefill_update_cache_extension",
            "load_mac_decode_rope_preserve_extension", "load_mac_merge_downdate_cache_extension")
_HOOK_MODULES = (
    "mac_attention.integrations.sglang.flashinfer_hooks",
    "mac_attention.integrations.sglang.llama_hooks",
)


def install(bridge_module: str = "mac_attention.integrations.sglang.bridge") -> list[str]:
    """Point the reference's loader names at this package.

    Call before the reference's hook modules are imported (they bind the loader
    names with ``from .bridge import ...``); modules that are already imported
    get the same names rebound.  All four loaders of the reference (decode,
    prefill update, RoPE-preserve, prefill downdate) are replaced.  Returns the
    names of the modules that were patched.
    """
    import importlib

    patched = []
    mod = importlib.import_module(bridge_module)
    for name in _PATCHED:
        setattr(mod, name, globals()[name])
    patched.append(bridge_module)
    for hook in _HOOK_MODULES:
        m = sys.modules.get(hook)
        if m is None:
            continue
        for name in _PATCHED:
            if hasattr(m, name):
                setattr(m, name, globals()[name])
        patched.append(hook)
    return patched
