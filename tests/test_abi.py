"""CPU: the C-ABI library builds for sm_100a, loads, and exports every symbol
that include/mac_b200.h declares (no compute calls without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

from mac_attention_b200 import _abi, build

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _abi.load_library()


def _declared_functions():
    text = (ROOT / "include" / "mac_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mac_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported(lib):
    names = _declared_functions()
    assert len(names) == 14
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_abi.PROTOTYPES) == names


def test_abi_version_and_error_text(lib):
    assert lib.mac_b200_abi_version() == _abi.ABI_VERSION
    assert lib.mac_b200_last_error() == b""
    assert lib.mac_b200_persistent_decode_bf16(None, None) == -1
    assert b"null" in lib.mac_b200_last_error()


def test_struct_layout_matches_c():
    from oracle import mac_oracle as O

    assert O.lib().mac_oracle_abi_struct_size() == ctypes.sizeof(_abi.MacB200DecodeArgs)
    assert O.lib().mac_oracle_build_struct_size() == ctypes.sizeof(_abi.MacB200PrefillBuildArgs)
    assert (O.lib().mac_oracle_build_struct_tail_offset()
            == _abi.MacB200PrefillBuildArgs.req_to_token.offset)


def test_argument_validation_needs_no_gpu(lib):
    a = _abi.MacB200DecodeArgs()
    a.D, a.Hq, a.Hkv = 64, 8, 2
    assert lib.mac_b200_persistent_decode_bf16(ctypes.byref(a), None) == -1
    assert b"D=128" in lib.mac_b200_last_error()
    a.D, a.Hq, a.Hkv = 128, 32, 2
    assert lib.mac_b200_persistent_decode_bf16(ctypes.byref(a), None) == -1
    assert b"GQA" in lib.mac_b200_last_error()
    p = _abi.MacB200PrefillArgs()
    assert lib.mac_b200_prefill_update_cache(ctypes.byref(p), None) == 0  # capacity 0: no-op
    p.M, p.B = 4, 1
    assert lib.mac_b200_prefill_update_cache(ctypes.byref(p), None) == -1


def test_torch_shim_builds_loads_and_keeps_the_reference_messages(lib):
    """The decode operator's torch-extension shim builds against this torch, links to the
    C-ABI library next to it, and raises the reference launcher's messages (checked here on
    CPU tensors, before anything touches a device)."""
    import torch

    from mac_attention_b200 import ops

    build.build_shim()
    shim = ops._load_shim()
    assert callable(shim.decode)
    t = torch.zeros(1, 8, 128, dtype=torch.bfloat16)
    args = [t] * 43 + [0] * 8 + [0.45, 0.088] + [0, 0] + [0.0] * 6 + [1, -1, 0] + [t] * 4
    assert len(args) == 68
    with pytest.raises(RuntimeError, match="q_post must be CUDA"):
        ops.mac_persistent_decode_bf16(*args)
    with pytest.raises(TypeError, match="68 positional"):
        ops.mac_persistent_decode_bf16(*args[:-1])
    with pytest.raises(TypeError):
        ops.mac_persistent_decode_bf16(*([None] + args[1:]))      # a required tensor is missing
