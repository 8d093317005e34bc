"""The reference's OWN kernel tests and checker, unmodified, against this library.

``oracle/build_ref.py`` stages the reference's ``attention/tests/
test_mac_persistent_decode.py``, its ``attention/tools/check_mac_persistent_decode.py``
(twelve checks), ``check_front_sink_recurrence.py`` and its loader module
``mac_attention/integrations/sglang/bridge.py`` byte for byte under
``oracle/_ref/ref_suite`` (git-ignored).  Here the reference's real loader module
is imported, :func:`mac_attention_b200.install` swaps its four loader functions,
and only then are the reference's test modules imported -- they bind the loader
with ``from mac_attention.integrations.sglang.bridge import ...`` exactly as the
reference's hooks do -- and run as they are.  Skipped where the suite was never
staged (no reference checkout at build time).
"""
import importlib
import importlib.util
import sys

import pytest
import torch

import mac_attention_b200
from oracle import build_ref

pytestmark = pytest.mark.gpu

TESTS = ["test_persistent_decode_hit_clean_half_open_cache_row",
         "test_persistent_decode_miss_multi_request",
         "test_persistent_decode_short_context_writes_empty_cache_row",
         "test_persistent_decode_tie_breaks_by_logical_position_after_wraparound"]
CHECKS = ["hit_clean_half_open_cache_row", "front_sink_rectification",
          "front_sink_mixed_group_exclusion", "front_sink_group4_mixed_fastpath",
          "front_sink_group4_full_fallback_reduce", "front_sink_group8_mixed_fastpath",
          "front_sink_group8_full_fallback_reduce", "miss_multi_request",
          "large_miss_reduced_rect", "mixed_group_reduced_rect", "short_context_empty_cache",
          "tie_break_after_wraparound"]


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def suite():
    root = build_ref.SUITE
    if not (root / "tests" / "test_mac_persistent_decode.py").exists():
        pytest.skip("the reference's suite was not staged for this box")
    sys.path.insert(0, str(root / "pkg"))
    try:
        ref_bridge = importlib.import_module("mac_attention.integrations.sglang.bridge")
        assert str(root) in ref_bridge.__file__           # the reference's own loader module
        patched = mac_attention_b200.install()
        assert "mac_attention.integrations.sglang.bridge" in patched
        tests = _load("ref_test_mac_persistent_decode", root / "tests" / "test_mac_persistent_decode.py")
        checks = _load("ref_check_mac_persistent_decode", root / "tools" / "check_mac_persistent_decode.py")
        # the names the reference modules bound at import are this library's loaders
        assert tests.load_mac_persistent_decode_extension is \
            mac_attention_b200.load_mac_persistent_decode_extension
        yield tests, checks, root
    finally:
        sys.path.remove(str(root / "pkg"))
        for name in [m for m in sys.modules if m == "mac_attention" or m.startswith("mac_attention.")]:
            del sys.modules[name]


@pytest.mark.parametrize("name", TESTS)
def test_reference_kernel_test_passes_unchanged(suite, name):
    tests, _, _ = suite
    getattr(tests, name)()
    assert mac_attention_b200.ops.query_status() == 0


@pytest.mark.parametrize("name", CHECKS)
def test_reference_checker_check_passes_unchanged(suite, name):
    _, checks, _ = suite
    ext = checks.load_mac_persistent_decode_extension(False)
    getattr(checks, f"_check_{name}")(ext)
    torch.cuda.synchronize()
    assert mac_attention_b200.ops.query_status() == 0


def test_reference_checker_main_and_recurrence_tool(suite, capsys):
    _, checks, root = suite
    checks.main()
    assert capsys.readouterr().out.count("PASS ") == len(CHECKS)
    recurrence = root / "tools" / "check_front_sink_recurrence.py"
    if recurrence.exists():
        mod = _load("ref_check_front_sink_recurrence", recurrence)   # two chained steps, F > 0
        with pytest.raises(SystemExit) as done:
            mod.main()
        assert done.value.code == 0, capsys.readouterr().out
    assert mac_attention_b200.ops.query_status() == 0
