"""Generate the golden vectors under ``tests/golden/`` from the reference itself.

Run where the reference checkout is mounted (it cannot travel to the GPU box):

    python tests/golden/make_golden.py [--reference <path of the reference checkout>]

What it imports from the reference and never re-implements:

* ``_ref_attention`` and ``_merge`` -- the PyTorch FP32 oracle helpers of
  ``attention/tools/check_mac_persistent_decode.py:9-51``;
* ``_synthetic_hit_and_slot`` -- the Python mirror of the kernel's synthetic
  benchmark decisions, ``benchmark/bench_mac_vs_flashinfer_direct.py:129-211``.

The decode cases follow the recipes of the reference's kernel tests and checker
(``attention/tests/test_mac_persistent_decode.py``, ``check_mac_persistent_decode.py:209-922``,
``check_front_sink_recurrence.py:52-134``): a match is planted in the ring at a
known position and the expected output / written ring row are composed from the
reference helpers exactly as those tests compose them.  Inputs are drawn on the
CPU with the seeds of the reference's cases (device RNG streams are not
portable, so the tensors are stored, not re-drawn).

Outputs: ``decode_cases.pt`` (list of dicts of CPU tensors + scalars) and
``bench_decisions.json``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def import_reference(root: Path):
    sys.path.insert(0, str(root / "attention"))
    sys.path.insert(0, str(root / "attention" / "src"))
    sys.path.insert(0, str(root / "benchmark"))
    from tools import check_mac_persistent_decode as chk  # noqa: E402

    try:
        import flashinfer  # noqa: F401
    except Exception:  # the benchmark script imports it at module scope only
        sys.modules["flashinfer"] = types.ModuleType("flashinfer")
    import bench_mac_vs_flashinfer_direct as bd  # noqa: E402

    return chk, bd


def pos_to_ring_slot(past_len, capacity, pos):
    if past_len < capacity:
        return pos
    slot = (pos - (past_len - capacity)) + past_len % capacity
    return slot - capacity if slot >= capacity else slot


def build_case(chk, *, name, seed, batch, hkv, group, capacity, kv_len, S, tile, mts, max_context,
               F=0, stride=64, hit_heads=None, match_pos=None, distinct_q=False, noise=0.0,
               far_cache=True, builder_query=False, cache_init="neg_inf", loc_dtype=torch.int32,
               extra_planted=None, tol_o=3e-2, tol_lse=3e-2, pins=None):
    """One single-step decode case.  ``hit_heads``: heads of every request whose
    ring holds a matching entry at ``match_pos``; other heads miss."""
    torch.manual_seed(seed)
    dt = torch.bfloat16
    dim = 128
    hq = hkv * group
    past = kv_len - 1
    sm = 1 / math.sqrt(dim)
    k = torch.randn(batch * kv_len, hkv, dim, dtype=dt)
    v = torch.randn_like(k)
    q_pre = torch.randn(batch, hq, dim, dtype=dt)
    q_post = torch.randn(batch, hq, dim, dtype=dt) if distinct_q else q_pre.clone()
    q_build = torch.randn(hq, dim, dtype=dt) if builder_query else None
    r2t = torch.zeros(batch, stride, dtype=torch.int32)
    ocl = torch.zeros(batch, dtype=loc_dtype)
    for n in range(batch):
        r2t[n, :past] = torch.arange(n * kv_len, n * kv_len + past, dtype=torch.int32)
        ocl[n] = n * kv_len + past
    req_ids = torch.arange(batch, dtype=torch.int32)
    past_lens = torch.full((batch,), past, dtype=torch.int32)
    qc = torch.randn(batch, capacity, hq, dim, dtype=dt)
    if far_cache:
        qc = (qc.float() + 10).to(dt)
    if cache_init == "neg_inf":
        ac = torch.zeros_like(qc)
        lc = torch.full((batch, capacity, hq), -float("inf"))
    else:  # stale finite garbage: must be overwritten, never reused
        ac = torch.ones_like(qc)
        lc = torch.zeros(batch, capacity, hq)

    new_end = max(past + 1 - S, 0)
    fs = min(F, new_end)
    hit_heads = list(hit_heads or [])
    exp_out = torch.zeros(batch, hq, dim, dtype=dt)
    exp_lse = torch.zeros(batch, hq)
    exp_ring_o = torch.zeros(batch, hq, dim, dtype=dt)
    exp_ring_lse = torch.zeros(batch, hq)
    exp_hit = torch.zeros(batch, hq, dtype=torch.int32)
    exp_mpos = torch.full((batch, hq), -1, dtype=torch.int32)

    for n in range(batch):
        kk = k[n * kv_len:(n + 1) * kv_len]
        vv = v[n * kv_len:(n + 1) * kv_len]
        entry_o = entry_l = None
        if hit_heads:
            mslot = pos_to_ring_slot(past, capacity, match_pos)
            pend = max(match_pos + 1 - S, 0)
            builder = q_build if q_build is not None else q_post[n]
            entry_o, entry_l = chk._ref_attention(builder, kk, vv, min(F, pend), pend, sm)
            for h in hit_heads:
                src = q_pre[n, h].float()
                if noise > 0:
                    src = src + noise * torch.randn(dim)
                qc[n, mslot, h] = src.to(dt)
                ac[n, mslot, h] = entry_o[h]
                lc[n, mslot, h] = entry_l[h]
        for pos, heads, kind in (extra_planted or []):
            # decoys: same query at another position with unusable state
            slot = pos_to_ring_slot(past, capacity, pos)
            for h in heads:
                qc[n, slot, h] = q_pre[n, h]
                if kind == "random_state":
                    ac[n, slot, h] = torch.randn(dim, dtype=dt)
                    lc[n, slot, h] = torch.randn(())
        full_o, full_l = chk._ref_attention(q_post[n], kk, vv, 0, kv_len, sm)
        miss_ring_o, miss_ring_l = chk._ref_attention(q_post[n], kk, vv, fs, new_end, sm)
        if hit_heads:
            pend = max(match_pos + 1 - S, 0)
            sink_o, sink_l = chk._ref_attention(q_post[n], kk, vv, 0, min(F, pend), sm)
            rect_o, rect_l = chk._ref_attention(q_post[n], kk, vv, pend, new_end, sm)
            tail_o, tail_l = chk._ref_attention(q_post[n], kk, vv, new_end, kv_len, sm)
            hc_o, hc_l = chk._merge(entry_o, entry_l, rect_o, rect_l)
            ho_o, ho_l = chk._merge(hc_o, hc_l, sink_o, sink_l)
            ho_o, ho_l = chk._merge(ho_o, ho_l, tail_o, tail_l)
        for h in range(hq):
            if h in hit_heads:
                exp_out[n, h], exp_lse[n, h] = ho_o[h], ho_l[h]
                exp_ring_o[n, h], exp_ring_lse[n, h] = hc_o[h], hc_l[h]
                exp_hit[n, h] = 1
                exp_mpos[n, h] = match_pos
            else:
                exp_out[n, h], exp_lse[n, h] = full_o[h], full_l[h]
                exp_ring_o[n, h], exp_ring_lse[n, h] = miss_ring_o[h], miss_ring_l[h]

    return {
        "name": name,
        "inputs": dict(q_post=q_post, q_pre=q_pre, k=k, v=v, req_to_token=r2t, req_ids=req_ids,
                       past_lens=past_lens, out_cache_loc=ocl, query_cache=qc, attn_cache=ac,
                       lse_cache=lc),
        "cfg": dict(max_context=max_context, tile_tokens=tile, match_tile_slots=mts,
                    semantic_pos_ahead=S, front_sink_tokens=F, threshold=0.45, sm_scale=sm),
        "expected": dict(out=exp_out, lse=exp_lse, ring_o=exp_ring_o, ring_lse=exp_ring_lse,
                         head_hit=exp_hit, head_match_pos=exp_mpos),
        "tol": dict(o=tol_o, lse=tol_lse),
        "pins": pins or {},
    }


def decode_cases(chk):
    cases = []
    # clean hit, half-open prefix (check.py:209-261; tests:100-191)
    cases.append(build_case(chk, name="hit_clean_half_open_cache_row", seed=1, batch=1, hkv=2,
                            group=4, capacity=8, kv_len=10, S=3, tile=4, mts=4, max_context=16,
                            hit_heads=range(8), match_pos=5, far_cache=False,
                            loc_dtype=torch.int64))
    # front sink, distinct pre/post queries, arbitrary builder (check.py:264-337)
    cases.append(build_case(chk, name="front_sink_rectification", seed=5, batch=1, hkv=2, group=4,
                            capacity=16, kv_len=20, S=4, tile=4, mts=4, max_context=32, F=3,
                            hit_heads=range(8), match_pos=10, distinct_q=True, noise=0.03,
                            builder_query=True, tol_o=7e-2, tol_lse=4e-2,
                            pins={"head_hit": True}))
    # GQA-8 mixed group 6 hit / 2 miss with front sink (check.py:340-446)
    cases.append(build_case(chk, name="front_sink_mixed_group_exclusion", seed=11, batch=1, hkv=1,
                            group=8, capacity=16, kv_len=20, S=4, tile=4, mts=4, max_context=32,
                            F=3, hit_heads=range(6), match_pos=10, distinct_q=True, noise=0.03,
                            builder_query=True, tol_o=8e-2, tol_lse=4e-2,
                            pins={"head_hit": True, "group_mode": [2]}))
    # mixed groups with a long band (check.py:460-570)
    cases.append(build_case(chk, name="front_sink_group4_mixed_fastpath", seed=13, batch=1, hkv=2,
                            group=4, capacity=16, kv_len=200, S=4, tile=4, mts=4, max_context=256,
                            F=6, stride=256, hit_heads=[0, 1, 4, 5, 6, 7], match_pos=190,
                            distinct_q=True, noise=0.03, builder_query=True, tol_o=8e-2,
                            tol_lse=4e-2, pins={"head_hit": True, "group_mode": [2, 0]}))
    cases.append(build_case(chk, name="front_sink_group8_mixed_fastpath", seed=13, batch=1, hkv=2,
                            group=8, capacity=16, kv_len=200, S=4, tile=4, mts=4, max_context=256,
                            F=6, stride=256, hit_heads=[0, 1, 2, 3] + list(range(8, 16)),
                            match_pos=190, distinct_q=True, noise=0.03, builder_query=True,
                            tol_o=8e-2, tol_lse=4e-2,
                            pins={"head_hit": True, "group_mode": [2, 0]}))
    # all-miss with front sink, long band (check.py:573-636)
    for g in (4, 8):
        cases.append(build_case(chk, name=f"front_sink_group{g}_full_fallback_reduce", seed=17,
                                batch=1, hkv=2, group=g, capacity=16, kv_len=300, S=4, tile=4,
                                mts=4, max_context=512, F=6, stride=512, tol_o=8e-2, tol_lse=4e-2,
                                pins={"head_hit": True, "group_mode": [1, 1]}))
    # multi-request all-miss (check.py:639-688; tests:194-278)
    cases.append(build_case(chk, name="miss_multi_request", seed=2, batch=2, hkv=2, group=4,
                            capacity=8, kv_len=12, S=4, tile=4, mts=4, max_context=16,
                            pins={"head_hit": True}))
    # large miss (check.py:690-734)
    cases.append(build_case(chk, name="large_miss_reduced_rect", seed=22, batch=1, hkv=2, group=4,
                            capacity=8, kv_len=192, S=4, tile=4, mts=4, max_context=256,
                            stride=256, pins={"head_hit": True, "task_counts3_positive": True}))
    # mixed group 3 hit / 1 miss without sink (check.py:737-816)
    cases.append(build_case(chk, name="mixed_group_reduced_rect", seed=23, batch=1, hkv=1, group=4,
                            capacity=8, kv_len=192, S=4, tile=4, mts=4, max_context=256,
                            stride=256, hit_heads=[0, 1, 3], match_pos=186, tol_o=8e-2,
                            pins={"head_hit": True, "group_mode": [2]}))
    # context shorter than S: ring row must be exactly (q, 0, -inf) (check.py:819-860)
    cases.append(build_case(chk, name="short_context_empty_cache", seed=3, batch=1, hkv=2, group=4,
                            capacity=8, kv_len=3, S=4, tile=4, mts=4, max_context=16, stride=32,
                            cache_init="stale", pins={"empty_ring_row": True}))
    # identical queries at two positions after wrap-around: older position wins
    # (check.py:863-922; tests:363-466)
    cases.append(build_case(chk, name="tie_break_after_wraparound", seed=4, batch=1, hkv=2, group=4,
                            capacity=4, kv_len=10, S=2, tile=4, mts=2, max_context=16, stride=32,
                            hit_heads=range(8), match_pos=6,
                            extra_planted=[(7, range(8), "random_state")],
                            pins={"head_hit": True, "head_match_pos": True}))
    return cases


def recurrence_case(chk):
    """Two chained steps, GQA-8: mixed write then all-hit reuse
    (check_front_sink_recurrence.py:52-134)."""
    torch.manual_seed(11)
    dt = torch.bfloat16
    hkv, group, dim = 1, 8, 128
    hq = hkv * group
    cap, S, tile, F, mts = 16, 4, 4, 3, 4
    sm = 1 / math.sqrt(dim)
    kv2, kv1 = 21, 20
    past1, past2 = kv1 - 1, kv1
    k = torch.randn(kv2, hkv, dim, dtype=dt)
    v = torch.randn_like(k)
    r2t = torch.zeros(1, 64, dtype=torch.int32)
    r2t[0, :past2] = torch.arange(past2, dtype=torch.int32)
    q_pre1 = torch.randn(1, hq, dim, dtype=dt)
    q_post1 = torch.randn(1, hq, dim, dtype=dt)
    q_build = torch.randn(hq, dim, dtype=dt)
    hit_heads = list(range(6))
    qc = (torch.randn(1, cap, hq, dim, dtype=dt).float() + 10).to(dt)
    ac = torch.zeros_like(qc)
    lc = torch.full((1, cap, hq), -float("inf"))
    mpos1 = 10
    mslot1 = mpos1 % cap
    pend1, nend1 = mpos1 + 1 - S, past1 + 1 - S
    entry_o, entry_l = chk._ref_attention(q_build, k, v, F, pend1, sm)
    for h in hit_heads:
        qc[0, mslot1, h] = (q_pre1[0, h].float() + 0.03 * torch.randn(dim)).to(dt)
        ac[0, mslot1, h] = entry_o[h]
        lc[0, mslot1, h] = entry_l[h]
    band1_o, band1_l = chk._ref_attention(q_post1[0], k, v, pend1, nend1, sm)
    e_hit_o, e_hit_l = chk._merge(entry_o, entry_l, band1_o, band1_l)
    e_miss_o, e_miss_l = chk._ref_attention(q_post1[0], k, v, F, nend1, sm)
    ring1_o = torch.stack([e_hit_o[h] if h in hit_heads else e_miss_o[h] for h in range(hq)])
    ring1_l = torch.stack([e_hit_l[h] if h in hit_heads else e_miss_l[h] for h in range(hq)])
    q_post2 = torch.randn(1, hq, dim, dtype=dt)
    nend2 = past2 + 1 - S
    sink2_o, sink2_l = chk._ref_attention(q_post2[0], k, v, 0, F, sm)
    rect2_o, rect2_l = chk._ref_attention(q_post2[0], k, v, nend1, nend2, sm)
    tail2_o, tail2_l = chk._ref_attention(q_post2[0], k, v, nend2, kv2, sm)
    ref2 = torch.zeros(hq, dim, dtype=dt)
    for h in range(hq):
        o, l = chk._merge(ring1_o[h:h + 1], ring1_l[h:h + 1], rect2_o[h:h + 1], rect2_l[h:h + 1])
        o, l = chk._merge(o, l, sink2_o[h:h + 1], sink2_l[h:h + 1])
        o, l = chk._merge(o, l, tail2_o[h:h + 1], tail2_l[h:h + 1])
        ref2[h] = o[0]
    return {
        "name": "front_sink_recurrence",
        "inputs": dict(k=k, v=v, req_to_token=r2t, req_ids=torch.tensor([0], dtype=torch.int32),
                       query_cache=qc, attn_cache=ac, lse_cache=lc,
                       q_pre1=q_pre1, q_post1=q_post1, q_post2=q_post2,
                       past1=past1, past2=past2),
        "cfg": dict(max_context=32, tile_tokens=tile, match_tile_slots=mts, semantic_pos_ahead=S,
                    front_sink_tokens=F, threshold=0.45, sm_scale=sm),
        "expected": dict(step1_head_hit=[1] * 6 + [0] * 2, ring1_o=ring1_o, ring1_lse=ring1_l,
                         step2_head_hit=[1] * hq, step2_match_pos=[past1] * hq, out2=ref2),
        "tol": dict(rel_l2=0.08),
    }


def bench_decisions(bd):
    """Expected synthetic decisions from the reference's Python mirror."""
    rows = []
    for mode in (1, 2):
        for batch, hq, hkv in ((1, 32, 8), (3, 32, 4), (5, 8, 1)):
            for past in (300, 65535):
                for capacity in (512, 2048):
                    for hit_rate in (0.0, 0.25, 0.5, 0.9, 1.0):
                        for std, skip, lag_std in ((0.0, -1.0, 0.0), (0.15, -1.0, 9.0),
                                                   (0.0, 0.7, 0.0)):
                            args = types.SimpleNamespace(
                                bench_seed=7, bench_hit_rate_std=std, capacity=capacity,
                                semantic_pos_ahead=256, bench_match_lag_mean=64.0,
                                bench_match_lag_std=lag_std, bench_skip_ratio=skip,
                                bench_skip_ratio_std=0.05 if skip >= 0 else 0.0)
                            hits, slots = [], []
                            group = hq // hkv
                            for n in range(batch):
                                for h in range(hq):
                                    hit, slot = bd._synthetic_hit_and_slot(
                                        args, bench_mode=mode, batch=batch, hq=hq, hkv=hkv,
                                        past_len=past, n=n, hq_i=h, hkv_i=h // group,
                                        hit_rate=hit_rate)
                                    hits.append("1" if hit else "0")
                                    slots.append(int(slot))
                            rows.append(dict(mode=mode, batch=batch, hq=hq, hkv=hkv, past=past,
                                             capacity=capacity, hit_rate=hit_rate, std=std,
                                             skip=skip, skip_std=args.bench_skip_ratio_std,
                                             lag_std=lag_std, seed=7, hits="".join(hits), slots=slots))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    a = ap.parse_args()
    chk, bd = import_reference(Path(a.reference))
    cases = decode_cases(chk)
    cases.append(recurrence_case(chk))
    torch.save(cases, HERE / "decode_cases.pt")
    with open(HERE / "bench_decisions.json", "w") as f:
        json.dump(bench_decisions(bd), f, separators=(",", ":"))
    print(f"wrote {len(cases)} decode cases and the bench decision table")


if __name__ == "__main__":
    main()
