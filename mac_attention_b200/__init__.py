"""B200-native MAC-Attention fused decode path.

The package is the host-side mirror of the reference's extension loader
(``attention/src/mac_attention/integrations/sglang/bridge.py`` in the reference
project): the same loader functions return objects with the same operator names
and positional signatures, backed by hand-written sm_100a CUDA kernels behind a
C ABI (``include/mac_b200.h``).  There is no CPU path: every operator raises
if the CUDA library is missing.
"""
from .bridge import (  # noqa: F401
    install,
    load_mac_decode_rope_preserve_extension,
    load_mac_merge_downdate_cache_extension,
    load_mac_persistent_decode_extension,
    load_mac_prefill_update_cache_extension,
)
from .workspace import make_decision_workspace, make_decode_workspace  # noqa: F401

__all__ = [
    "install",
    "load_mac_decode_rope_preserve_extension",
    "load_mac_merge_downdate_cache_extension",
    "load_mac_persistent_decode_extension",
    "load_mac_prefill_update_cache_extension",
    "make_decision_workspace",
    "make_decode_workspace",
]
