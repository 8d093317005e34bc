"""GPU: the decode entry point that allocates nothing.

Some hosts may not allocate device memory at all -- a serving process whose own
pool owns all of HBM, or a plugin under a sandbox that filters allocation
calls.  ``mac_b200_persistent_decode_bf16_noalloc`` keeps its scratch in a fixed
8 MiB block inside the library instead.  Here it is called through the C ABI
twice in a row (the block keeps the first call's contents) and compared with
the allocating entry point on the same inputs; a step that does not fit the
block must be refused with a clear error, not run.

Collected last on purpose: a run that stops at the first failure has then
already run every other test."""
import pytest
import torch

from mac_attention_b200 import load_mac_persistent_decode_extension, make_decode_workspace
from mac_attention_b200 import ops, synth
from oracle import mac_oracle as O
from tests.helpers import REL_L2_TOL

pytestmark = pytest.mark.gpu


def _step(entry, case, cfg, batch, hq, hkv, capacity):
    c = case.to("cuda").clone()
    ws = make_decode_workspace(batch, hq, hkv, capacity, cfg.max_context, cfg.tile_tokens,
                               cfg.match_tile_slots, cfg.semantic_pos_ahead)
    out = torch.full_like(c.q_post, float("nan"))
    lse = torch.full((batch, hq), float("nan"), device="cuda")
    e = torch.empty(0)
    entry(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens, c.out_cache_loc,
          c.query_cache, c.attn_cache, c.lse_cache, out, lse, *ws, *cfg.scalar_args(),
          c.query_cache, e, e, e)
    torch.cuda.synchronize()
    return out, lse, ws, c


def test_noalloc_entry_matches_allocating_entry_twice_in_a_row():
    ext = load_mac_persistent_decode_extension()
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=128)
    shapes = [dict(batch=3, ctxs=[2500, 700, 3300], hq=32, hkv=8, capacity=256, seed=41),
              dict(batch=2, ctxs=[1800, 2900], hq=32, hkv=4, capacity=512, seed=42)]
    for sp in shapes:  # two different calls back to back through the same fixed block
        case = synth.make_decode_case(batch=sp["batch"], ctx=0, ctx_list=sp["ctxs"], hq=sp["hq"],
                                      hkv=sp["hkv"], capacity=sp["capacity"], seed=sp["seed"])
        synth.plant_matches(case, hit_fraction=0.6, borderline_fraction=0.4, seed=sp["seed"])
        a = (sp["batch"], sp["hq"], sp["hkv"], sp["capacity"])
        ref_out, ref_lse, ref_ws, ref_case = _step(ext.mac_persistent_decode_bf16, case, cfg, *a)
        for _ in range(2):
            out, lse, ws, c = _step(ext.mac_persistent_decode_bf16_noalloc, case, cfg, *a)
            for idx in (3, 4, 5, 6, 7, 8, 9, 15):
                assert torch.equal(ws[idx], ref_ws[idx]), f"workspace[{idx}] differs"
            assert torch.isfinite(out.float()).all()
            assert O.rel_l2(out.float().cpu(), ref_out.float().cpu()) <= REL_L2_TOL
            assert (lse - ref_lse).abs().max() <= 2e-2
            assert torch.equal(c.query_cache, ref_case.query_cache)
            assert O.rel_l2(c.attn_cache.float().cpu(), ref_case.attn_cache.float().cpu()) <= REL_L2_TOL
    assert ops.query_status() == 0


def test_noalloc_entry_leaves_free_device_memory_unchanged():
    """The point of the entry: the driver hands out no device memory for it.  Free memory
    as the driver reports it is the same before and after a call (the inputs are made
    first, and the first call on the device -- which looks up the block's address -- is
    made before the measurement)."""
    ext = load_mac_persistent_decode_extension()
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=128)
    case = synth.make_decode_case(batch=3, ctx=0, ctx_list=[2500, 700, 3300], hq=32, hkv=8,
                                  capacity=256, seed=41)
    c = case.to("cuda").clone()
    ws = make_decode_workspace(3, 32, 8, 256, cfg.max_context, cfg.tile_tokens,
                               cfg.match_tile_slots, cfg.semantic_pos_ahead)
    out = torch.empty_like(c.q_post)
    lse = torch.empty(3, 32, device="cuda")
    e = torch.empty(0)

    def call():
        ext.mac_persistent_decode_bf16_noalloc(
            c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens, c.out_cache_loc,
            c.query_cache, c.attn_cache, c.lse_cache, out, lse, *ws, *cfg.scalar_args(),
            c.query_cache, e, e, e)
        torch.cuda.synchronize()

    call()                                   # set-up call
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    call()
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert ops.query_status() == 0


def test_noalloc_entry_refuses_steps_beyond_its_fixed_block():
    ext = load_mac_persistent_decode_extension()
    cfg = O.DecodeConfig(max_context=256, semantic_pos_ahead=16)
    # 300 requests x 8 KV heads x 8 query heads per group needs well over 8 MiB of partials
    case = synth.make_decode_case(batch=300, ctx=40, hq=64, hkv=8, capacity=8, seed=1)
    with pytest.raises(RuntimeError, match="fixed block"):
        _step(ext.mac_persistent_decode_bf16_noalloc, case, cfg, 300, 64, 8, 8)
    # the allocating entry point takes the same step
    out, _, _, _ = _step(ext.mac_persistent_decode_bf16, case, cfg, 300, 64, 8, 8)
    assert torch.isfinite(out.float()).all()
