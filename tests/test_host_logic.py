"""CPU: host-side mirror of the reference's loader/operator interface."""
import sys
import types

import pytest
import torch

import mac_attention_b200 as pkg
from mac_attention_b200 import bridge, ops, sharding, synth, workspace
from oracle import mac_oracle as O


def test_loaders_expose_reference_operator_names():
    dec = pkg.load_mac_persistent_decode_extension(False, fast_math=True)
    assert callable(dec.mac_persistent_decode_bf16)
    pre = pkg.load_mac_prefill_update_cache_extension(False)
    for name in ("mac_prefill_update_cache", "mac_mark_persistent_ready",
                 "mac_invalidate_persistent_ready", "mac_update_request_state"):
        assert callable(getattr(pre, name))
    assert callable(pkg.load_mac_decode_rope_preserve_extension().mac_decode_rope_preserve_q_bf16)
    assert callable(
        pkg.load_mac_merge_downdate_cache_extension().mac_update_then_downdate_bf16_inplace)
    assert pkg.load_mac_persistent_decode_extension(False, fast_math=True) is dec


def test_install_rebinds_bridge_and_imported_hooks(monkeypatch):
    fake_bridge = types.ModuleType("fake_mac.bridge")
    fake_bridge.load_mac_persistent_decode_extension = lambda *a, **k: "old"
    fake_bridge.load_mac_prefill_update_cache_extension = lambda *a, **k: "old"
    fake_bridge.load_mac_decode_rope_preserve_extension = lambda *a, **k: "rope"
    monkeypatch.setitem(sys.modules, "fake_mac", types.ModuleType("fake_mac"))
    monkeypatch.setitem(sys.modules, "fake_mac.bridge", fake_bridge)
    hooks = types.ModuleType("mac_attention.integrations.sglang.flashinfer_hooks")
    hooks.load_mac_persistent_decode_extension = fake_bridge.load_mac_persistent_decode_extension
    monkeypatch.setitem(sys.modules, "mac_attention.integrations.sglang.flashinfer_hooks", hooks)
    patched = bridge.install("fake_mac.bridge")
    assert "fake_mac.bridge" in patched and hooks.__name__ in patched
    assert fake_bridge.load_mac_persistent_decode_extension is bridge.load_mac_persistent_decode_extension
    assert hooks.load_mac_persistent_decode_extension is bridge.load_mac_persistent_decode_extension
    assert fake_bridge.load_mac_decode_rope_preserve_extension is bridge.load_mac_decode_rope_preserve_extension
    assert fake_bridge.load_mac_merge_downdate_cache_extension is bridge.load_mac_merge_downdate_cache_extension


def test_install_patches_the_reference_loader_module_itself():
    """The reference's real ``bridge`` module (from the staged copy of its loader, or from
    its checkout) is imported, ``install()`` is called on it, and all four loader names --
    also in a module that had bound them at import, the way the reference's hook modules
    do -- resolve to this library and return objects with the pybind operator names."""
    import importlib
    import os
    from pathlib import Path

    from oracle import build_ref

    roots = [build_ref.SUITE / "pkg",
             Path(os.environ.get("MAC_REFERENCE_ROOT", "/root/reference")) / "attention" / "src"]
    root = next((r for r in roots
                 if (r / "mac_attention" / "integrations" / "sglang" / "bridge.py").exists()), None)
    if root is None:
        pytest.skip("no copy of the reference's loader module on this machine")
    staged = root == roots[0]
    sys.path.insert(0, str(root))
    try:
        if not staged:   # the checkout's package __init__ imports the SGLang hooks
            for name in ("mac_attention", "mac_attention.integrations",
                         "mac_attention.integrations.sglang"):
                m = types.ModuleType(name)
                m.__path__ = [str(root / name.replace(".", "/"))]
                sys.modules[name] = m
        ref_bridge = importlib.import_module("mac_attention.integrations.sglang.bridge")
        early = types.ModuleType("mac_attention.integrations.sglang.llama_hooks")
        for name in bridge._PATCHED:          # bound before install(), as the hook modules do
            setattr(early, name, getattr(ref_bridge, name))
        sys.modules[early.__name__] = early
        originals = {name: getattr(ref_bridge, name) for name in bridge._PATCHED}
        patched = bridge.install()
        assert patched[0] == "mac_attention.integrations.sglang.bridge" and early.__name__ in patched
        for name in bridge._PATCHED:
            assert getattr(ref_bridge, name) is getattr(bridge, name) is getattr(early, name)
            assert getattr(ref_bridge, name) is not originals[name]
        dec = ref_bridge.load_mac_persistent_decode_extension(False)
        assert callable(dec.mac_persistent_decode_bf16)
        pre = ref_bridge.load_mac_prefill_update_cache_extension(False)
        for op in ("mac_prefill_update_cache", "mac_mark_persistent_ready",
                   "mac_invalidate_persistent_ready", "mac_update_request_state"):
            assert callable(getattr(pre, op))
        assert callable(ref_bridge.load_mac_decode_rope_preserve_extension().mac_decode_rope_preserve_q_bf16)
        assert callable(
            ref_bridge.load_mac_merge_downdate_cache_extension().mac_update_then_downdate_bf16_inplace)
    finally:
        sys.path.remove(str(root))
        for name in [m for m in sys.modules if m == "mac_attention" or m.startswith("mac_attention.")]:
            del sys.modules[name]


def test_decode_operator_rejects_cpu_tensors_like_the_reference():
    case = synth.make_decode_case(batch=1, ctx=20, hq=8, hkv=2, capacity=8, seed=0)
    cfg = O.DecodeConfig(max_context=32, semantic_pos_ahead=4)
    ws = workspace.make_decode_workspace(1, 8, 2, 8, 32, 32, 32, 4, device="cpu")
    out = torch.empty_like(case.q_post)
    e = torch.empty(0)
    with pytest.raises(RuntimeError, match="q_post must be CUDA"):
        ops.mac_persistent_decode_bf16(case.q_post, case.q_pre, case.k, case.v, case.req_to_token,
                                       case.req_ids, case.past_lens, case.out_cache_loc,
                                       case.query_cache, case.attn_cache, case.lse_cache, out,
                                       torch.empty(1, 8), *ws, *cfg.scalar_args(),
                                       case.query_cache, e, e, e)
    assert len(ws) == 30 and len(cfg.scalar_args()) == 21


def test_workspace_shapes_follow_the_reference_callers():
    ws = workspace.make_decode_workspace(3, 32, 8, 2048, 131072, 32, 32, 256, 64, device="cpu",
                                         partial_dtype=torch.bfloat16)
    assert tuple(ws[0].shape) == (3, 32, 64)
    assert tuple(ws[workspace.GROUP_MODE].shape) == (3, 8)
    assert ws[workspace.TASK_COUNTS].numel() == 9
    assert tuple(ws[23].shape) == (3, 8, 4098, 4, 128) and ws[23].dtype == torch.bfloat16
    assert ws[16].numel() == 3 * 32 * 4098 and ws[workspace.PHASE_CYCLES].dtype == torch.int64


def test_prefill_noop_paths_do_not_need_the_device():
    z = torch.zeros(0, dtype=torch.int32)
    assert ops.mac_prefill_update_cache(None, None, None, None, z, None, None, None, None, None,
                                        0, 4, 128, None) is None
    assert ops.mac_mark_persistent_ready(None, None, None, z) is None


def test_kv_head_shards_reassemble_the_unsharded_step():
    case = synth.make_decode_case(batch=2, ctx=300, hq=16, hkv=4, capacity=64, seed=3)
    synth.plant_matches(case, hit_fraction=0.5, seed=1)
    cfg = O.DecodeConfig(max_context=512, semantic_pos_ahead=32)
    full_case = case.clone()
    full = O.decode_step(full_case.q_post, full_case.q_pre, full_case.k, full_case.v,
                         full_case.req_to_token, full_case.req_ids, full_case.past_lens,
                         full_case.out_cache_loc, full_case.query_cache, full_case.attn_cache,
                         full_case.lse_cache, cfg)
    outs, hits, rings = [], [], []
    for r in range(2):
        sh = sharding.shard_case(case, 2, r)
        res = O.decode_step(sh.q_post, sh.q_pre, sh.k, sh.v, sh.req_to_token, sh.req_ids,
                            sh.past_lens, sh.out_cache_loc, sh.query_cache, sh.attn_cache,
                            sh.lse_cache, cfg)
        outs.append(res.out)
        hits.append(res.head_hit)
        rings.append(sh.attn_cache)
    assert torch.equal(sharding.gather_heads(outs), full.out)
    assert torch.equal(sharding.gather_heads(hits), full.head_hit)
    assert torch.equal(sharding.gather_heads(rings, dim=2), full_case.attn_cache)
    with pytest.raises(ValueError):
        sharding.head_slices(16, 4, 3, 0)


def test_one_pass_prefill_build_host_checks_need_no_device():
    """No-op paths return before touching the device; wrong placements and shapes raise the
    operator's messages from the host-side checks."""
    import pytest

    from mac_attention_b200 import load_mac_prefill_update_cache_extension

    ext = load_mac_prefill_update_cache_extension()
    assert hasattr(ext, "mac_prefill_downdate_update_cache")
    R, M, H, D, rows = 2, 4, 2, 128, 3
    t = dict(q=torch.zeros(R, M, H, D, dtype=torch.bfloat16), a=torch.zeros(R, M, H, D, dtype=torch.bfloat16),
             l=torch.zeros(R, M, H), rl=torch.zeros(R, dtype=torch.int32),
             ids=torch.zeros(1, dtype=torch.int32), sq=torch.zeros(rows, H, D, dtype=torch.bfloat16),
             fl=torch.zeros(rows, H), off=torch.tensor([0, rows], dtype=torch.int32),
             ln=torch.tensor([rows], dtype=torch.int32))

    def call(capacity=M, ids=None):
        ext.mac_prefill_downdate_update_cache(t["q"], t["a"], t["l"], t["rl"],
                                              t["ids"] if ids is None else ids, t["sq"], t["sq"],
                                              t["fl"], t["sq"], t["fl"], t["off"], t["ln"],
                                              capacity, H, D, None)

    call(capacity=0)                                      # silent no-op, as the reference's copy
    call(ids=torch.zeros(0, dtype=torch.int32))           # empty batch
    with pytest.raises(RuntimeError, match="must be CUDA"):
        call()
