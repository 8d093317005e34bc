"""The bench's parity leg, exercised on the CPU: the oracle restricted to a
sample of rows must reproduce its own full-batch results on those rows, and
``bench.parity_sample`` (compact host pool, remapped page table and ring) must
report a clean record when the "device" results are the oracle's own."""
import argparse

import torch

import bench
from mac_attention_b200 import synth
from mac_attention_b200 import workspace as W
from oracle import mac_oracle as O


def _case(front_sink=0):
    case = synth.make_decode_case(batch=6, ctx=0, ctx_list=[700, 1500, 900, 2100, 650, 1200], hq=8,
                                  hkv=2, capacity=256, page_size=16, seed=3,
                                  sink_boost=64 if front_sink else 0)
    return case


def _cfg(front_sink=0, hit=0.6):
    return O.DecodeConfig(max_context=bench.MAX_CONTEXT, tile_tokens=bench.TILE,
                          match_tile_slots=bench.MTS, semantic_pos_ahead=bench.SEM,
                          front_sink_tokens=front_sink, bench_mode=1, bench_hit_rate=hit,
                          bench_match_lag_mean=float(bench.LAG), bench_seed=1)


def _full(case, cfg):
    c = case.clone()
    res = O.decode_step(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens,
                        c.out_cache_loc, c.query_cache, c.attn_cache, c.lse_cache, cfg)
    return res, c


def test_row_mask_reproduces_full_batch_rows():
    case, cfg = _case(), _cfg()
    full, _ = _full(case, cfg)
    mask = torch.tensor([1, 0, 0, 1, 1, 0], dtype=torch.uint8)
    c = case.clone()
    part = O.decode_step(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens,
                         c.out_cache_loc, c.query_cache, c.attn_cache, c.lse_cache, cfg,
                         row_mask=mask)
    rows = mask.bool()
    for name in ("head_hit", "head_match_pos", "head_rect_start", "group_mode", "out", "lse"):
        assert torch.equal(getattr(part, name)[rows], getattr(full, name)[rows]), name
    assert not part.out[~rows].float().abs().any()
    # rows left out do not write their ring row
    untouched = case.query_cache[1, int(case.past_lens[1]) % 256]
    assert torch.equal(c.query_cache[1, int(case.past_lens[1]) % 256], untouched)


def test_parity_sample_is_clean_on_the_oracles_own_results():
    for front_sink in (0, 64):
        case, cfg = _case(front_sink), _cfg(front_sink)
        full, after = _full(case, cfg)
        N, hq, hkv = 6, 8, 2
        ws = [None] * 30
        for idx, name in ((W.HEAD_HIT, "head_hit"), (W.HEAD_MATCH_SLOT, "head_match_slot"),
                          (W.HEAD_MATCH_POS, "head_match_pos"), (W.HEAD_PREFIX_END, "head_prefix_end"),
                          (W.HEAD_RECT_START, "head_rect_start"), (W.HEAD_NEW_END, "head_new_end"),
                          (W.GROUP_RECT_BEGIN, "group_rect_begin"), (W.GROUP_MODE, "group_mode")):
            ws[idx] = getattr(full, name)
        args = argparse.Namespace(bench_mode=1, hit=0.6, batch=N)
        ab = bench.alg_bytes(ws, N, hq, hkv, front_sink, 256, case.past_lens.tolist())
        # the "device" state after the step: ring rows written, outputs of the full run
        parity, secs, share = bench.parity_sample(args, after, ws, full.out, full.lse, ab["per_row"],
                                                  hq, hkv, front_sink, max_rows=4)
        assert parity["ok"], parity
        assert parity["requests_checked"] == 4 and parity["decisions_equal"]
        assert 0 < share <= 1 and secs > 0
        assert parity["out_rel_l2"] < 5e-3      # bf16 rounding of the stored output only
        # a corrupted output row is caught
        bad = full.out.clone()
        bad[parity["rows"][0]] = 0
        parity2, _, _ = bench.parity_sample(args, after, ws, bad, full.lse, ab["per_row"], hq, hkv,
                                            front_sink, max_rows=4)
        assert not parity2["ok"]
