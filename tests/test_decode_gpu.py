"""GPU parity of the fused decode step: CUDA kernel (through the C ABI) against
the golden vectors, the CPU oracle and, when it was built, the reference's own
CUDA kernel compiled for sm_100a."""
import math
import os

import pytest
import torch

from mac_attention_b200 import load_mac_persistent_decode_extension, make_decode_workspace
from mac_attention_b200 import ops, synth
from oracle import mac_oracle as O
from tests.helpers import (REL_L2_TOL, assert_decisions_equal, assert_outputs_close,
                           case_from_golden, ring_rows, run_cuda, run_oracle)

pytestmark = pytest.mark.gpu

GOLDEN_NAMES = [
    "hit_clean_half_open_cache_row", "front_sink_rectification",
    "front_sink_mixed_group_exclusion", "front_sink_group4_mixed_fastpath",
    "front_sink_group8_mixed_fastpath", "front_sink_group4_full_fallback_reduce",
    "front_sink_group8_full_fallback_reduce", "miss_multi_request", "large_miss_reduced_rect",
    "mixed_group_reduced_rect", "short_context_empty_cache", "tie_break_after_wraparound",
]


def _status_clean():
    assert ops.query_status() == 0


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_golden_cases(golden_cases, name):
    g = next(c for c in golden_cases if c["name"] == name)
    case = case_from_golden(g)
    cfg = O.DecodeConfig(**g["cfg"])
    cu = run_cuda(case, cfg, partial_dtype=torch.bfloat16)
    orc, orc_case = run_oracle(case, cfg)
    N = case.q_post.shape[0]
    assert_decisions_equal(cu, orc, N)
    assert_outputs_close(cu, orc, orc_case)
    # the reference's own assertions on its own expected values
    e, tol = g["expected"], g["tol"]
    torch.testing.assert_close(cu.out.cpu().float(), e["out"].float(), rtol=tol["o"], atol=tol["o"])
    torch.testing.assert_close(cu.lse.cpu(), e["lse"], rtol=tol["lse"], atol=tol["lse"])
    assert torch.equal(cu.ws[3][:N].cpu(), e["head_hit"])
    assert torch.equal(cu.ws[5][:N].cpu(), e["head_match_pos"])
    q_row, o_row, l_row = ring_rows(cu.case.to("cpu"))
    fin = torch.isfinite(e["ring_lse"])
    if fin.any():
        torch.testing.assert_close(o_row.float()[fin], e["ring_o"].float()[fin], rtol=tol["o"],
                                   atol=tol["o"])
        torch.testing.assert_close(l_row[fin], e["ring_lse"][fin], rtol=tol["lse"], atol=tol["lse"])
    pins = g["pins"]
    if "group_mode" in pins:
        assert cu.ws[15][:N].flatten().tolist() == pins["group_mode"]
    if pins.get("task_counts3_positive"):
        assert int(cu.ws[22][3]) > 0
    if pins.get("empty_ring_row"):
        assert torch.equal(q_row, case.q_pre)
        assert torch.equal(o_row, torch.zeros_like(o_row))
        assert torch.isneginf(l_row).all()
    _status_clean()


def test_two_step_recurrence(golden_cases):
    g = next(c for c in golden_cases if c["name"] == "front_sink_recurrence")
    i, e = g["inputs"], g["expected"]
    cfg = O.DecodeConfig(**g["cfg"])
    p1 = torch.tensor([i["past1"]], dtype=torch.int32)
    c1 = synth.DecodeCase(q_post=i["q_post1"], q_pre=i["q_pre1"], k=i["k"], v=i["v"],
                          req_to_token=i["req_to_token"], req_ids=i["req_ids"], past_lens=p1,
                          out_cache_loc=p1.clone(), query_cache=i["query_cache"],
                          attn_cache=i["attn_cache"], lse_cache=i["lse_cache"])
    r1 = run_cuda(c1, cfg)
    assert r1.ws[3][0].tolist() == e["step1_head_hit"]
    M = c1.query_cache.shape[1]
    assert O.rel_l2(r1.case.attn_cache[0, i["past1"] % M].float().cpu(), e["ring1_o"].float()) < 1e-2
    p2 = torch.tensor([i["past2"]], dtype=torch.int32)
    c2 = r1.case.clone()
    c2.q_post, c2.past_lens, c2.out_cache_loc = i["q_post2"], p2, p2.clone()
    r2 = run_cuda(c2, cfg)
    assert r2.ws[3][0].tolist() == e["step2_head_hit"]
    assert r2.ws[5][0].tolist() == e["step2_match_pos"]
    assert O.rel_l2(r2.out[0].float().cpu(), e["out2"].float()) < 1.5e-2
    _status_clean()


CASES = [
    # batch, ctx list, hq, hkv, capacity, S, F, mts, page, seed
    dict(batch=3, ctxs=[3000, 777, 4500], hq=32, hkv=8, capacity=512, S=256, F=0, mts=32, page=16),
    dict(batch=2, ctxs=[2100, 5000], hq=32, hkv=4, capacity=512, S=256, F=64, mts=32, page=16),
    dict(batch=4, ctxs=[300, 40, 1300, 2], hq=16, hkv=2, capacity=128, S=64, F=128, mts=32, page=1),
    dict(batch=2, ctxs=[1500, 900], hq=8, hkv=8, capacity=256, S=100, F=0, mts=16, page=16),
    dict(batch=2, ctxs=[1200, 640], hq=28, hkv=4, capacity=200, S=256, F=3, mts=24, page=8),
    dict(batch=1, ctxs=[6000], hq=64, hkv=8, capacity=1024, S=256, F=0, mts=32, page=16),
]


@pytest.mark.parametrize("spec", CASES, ids=lambda s: f"b{s['batch']}_hq{s['hq']}_hkv{s['hkv']}_F{s['F']}")
def test_planted_and_borderline_matches_vs_oracle(spec):
    case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"], hq=spec["hq"],
                                  hkv=spec["hkv"], capacity=spec["capacity"],
                                  page_size=spec["page"], seed=31, kv_scale=1.0)
    synth.plant_matches(case, hit_fraction=0.5, noise=0.1, borderline_fraction=0.6, seed=5,
                        lag_hi=spec["capacity"])
    cfg = O.DecodeConfig(max_context=8192, semantic_pos_ahead=spec["S"],
                         front_sink_tokens=spec["F"], match_tile_slots=spec["mts"])
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, spec["batch"])
    # per-tile scan results: identical wherever a candidate beat the threshold
    thr = O.threshold_distance(cfg.threshold)
    md, mp, ms = cu.ws[0].cpu(), cu.ws[1].cpu(), cu.ws[2].cpu()
    sel = orc.match_dist < thr
    assert torch.equal(md[sel], orc.match_dist[sel])
    assert torch.equal(mp[sel], orc.match_pos[sel]) and torch.equal(ms[sel], orc.match_slot[sel])
    assert_outputs_close(cu, orc, orc_case)
    assert 0 < int(orc.head_hit.sum()) < orc.head_hit.numel()
    _status_clean()


def test_probe_never_drops_rows_whose_distance_sits_in_the_probed_half():
    """Ring rows that differ from the query only in the first 64 dims, with a
    squared distance within 3 % of the threshold on either side: the scan's
    approximate probe sees the whole distance, so this is where a too tight
    pruning margin would flip a decision."""
    case = synth.make_decode_case(batch=2, ctx=3000, hq=32, hkv=8, capacity=512, seed=23)
    g = torch.Generator().manual_seed(99)
    thr = 2.0 * 128 * (1.0 - 0.45) ** 2
    for n in range(2):
        P = int(case.past_lens[n])
        for h in range(32):
            for rep in range(3):
                pos = P - 1 - int(torch.randint(0, 500, (1,), generator=g))
                d = torch.zeros(128)
                d[:64] = torch.randn(64, generator=g)
                tgt = thr * (0.97 + 0.06 * float(torch.rand((), generator=g)))
                row = case.q_pre[n, h].float() + d * math.sqrt(tgt / float((d * d).sum()))
                case.query_cache[n, pos % 512, h] = row.to(torch.bfloat16)
                case.lse_cache[n, pos % 512, h] = 3.0
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=64)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 2)
    assert 5 < int(orc.head_hit.sum()) < 64
    assert_outputs_close(cu, orc, orc_case)
    _status_clean()


def test_config0_shape_cpu_plumbing_case():
    """Llama-3.1-8B attention shape, batch 2, context 4096, 64 planted prior
    queries, half of the step queries near a planted one."""
    case = synth.make_decode_case(batch=2, ctx=4096, hq=32, hkv=8, capacity=4096, page_size=16,
                                  seed=0, kv_scale=1.0 / math.sqrt(128))
    synth.plant_matches(case, hit_fraction=0.5, noise=0.1, lag_lo=256, lag_hi=4096, seed=0)
    cfg = O.DecodeConfig(max_context=8192, semantic_pos_ahead=256)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 2)
    assert_outputs_close(cu, orc, orc_case)
    _status_clean()


def test_readiness_gate_demotes_without_touching_ring():
    case = synth.make_decode_case(batch=6, ctx=0, ctx_list=[900, 1200, 500, 2000, 1500, 700],
                                  hq=32, hkv=8, capacity=256, page_size=16, seed=9, ring_rows=9,
                                  req_ids=[8, 3, 0, 5, 1, 7])
    synth.plant_matches(case, hit_fraction=0.8, seed=2)
    synth.add_readiness_gate(case, not_ready_fraction=0.3, stale_fraction=0.25, seed=3)
    off = case.meta["gated_off"]
    assert off[case.req_ids.long()].any() and not off[case.req_ids.long()].all()
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=64)
    before = case.clone()
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 6)
    assert_outputs_close(cu, orc, orc_case)
    after = cu.case.to("cpu")
    M = case.query_cache.shape[1]
    for n in range(6):
        req, P = int(case.req_ids[n]), int(case.past_lens[n])
        if off[req]:
            assert cu.ws[3][n].sum() == 0 and (cu.ws[15][n] == 1).all()
            assert torch.equal(after.query_cache[req], before.query_cache[req])
            assert torch.equal(after.attn_cache[req], before.attn_cache[req])
            assert torch.equal(after.lse_cache[req], before.lse_cache[req])
        else:
            assert torch.equal(after.query_cache[req, P % M], case.q_pre[n])
    _status_clean()


@pytest.mark.parametrize("mode,hit_rate,std,skip", [(1, 0.9, 0.0, -1.0), (2, 0.75, 0.0, -1.0),
                                                    (1, 0.5, 0.2, -1.0), (1, 0.8, 0.0, 0.6),
                                                    (1, 1.0, 0.0, -1.0), (1, 0.0, 0.0, -1.0)])
def test_synthetic_bench_decisions_and_outputs(mode, hit_rate, std, skip):
    case = synth.make_decode_case(batch=5, ctx=0, ctx_list=[3000, 2500, 3100, 1800, 2700], hq=32,
                                  hkv=8, capacity=512, page_size=16, seed=4)
    cfg = O.DecodeConfig(max_context=4096, bench_mode=mode, bench_hit_rate=hit_rate,
                         bench_hit_rate_std=std, bench_skip_ratio=skip, bench_match_lag_std=3.0,
                         bench_seed=11, bench_layer_id=3)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 5)
    assert_outputs_close(cu, orc, orc_case)
    _status_clean()


def test_miss_mask_and_mixed_group_switch(monkeypatch):
    case = synth.make_decode_case(batch=2, ctx=1500, hq=32, hkv=4, capacity=256, seed=8)
    for mixed in ("1", "0"):
        monkeypatch.setenv("MAC_PERSISTENT_MIXED_GROUP_FALLBACK", mixed)
        cfg = O.DecodeConfig(max_context=2048, bench_miss_mask=0b00100101,
                             mixed_group_fallback=int(mixed))
        cu = run_cuda(case, cfg)
        orc, orc_case = run_oracle(case, cfg)
        assert_decisions_equal(cu, orc, 2)
        assert_outputs_close(cu, orc, orc_case)
        assert (cu.ws[15][:2] == (2 if mixed == "1" else 1)).all()
    _status_clean()


def test_oversized_workspace_int64_loc_and_no_lse():
    case = synth.make_decode_case(batch=3, ctx=700, hq=16, hkv=4, capacity=64, seed=12,
                                  loc_dtype=torch.int64)
    synth.plant_matches(case, hit_fraction=0.6, seed=1)
    cfg = O.DecodeConfig(max_context=1024, semantic_pos_ahead=32)
    cu = run_cuda(case, cfg, ws_batch=7)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 3)
    assert_outputs_close(cu, orc, orc_case)
    # rows beyond N stay untouched (poison value)
    assert (cu.ws[3][3:] == -7).all()
    # optional_lse may be an empty tensor
    ext = load_mac_persistent_decode_extension()
    c = case.to("cuda")
    ws = make_decode_workspace(3, 16, 4, 64, 1024, 32, 32, 32)
    out = torch.empty_like(c.q_post)
    e = torch.empty(0)
    ext.mac_persistent_decode_bf16(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids,
                                   c.past_lens, c.out_cache_loc, c.query_cache, c.attn_cache,
                                   c.lse_cache, out, torch.empty(0, device="cuda"), *ws,
                                   *cfg.scalar_args(), c.query_cache, e, e, e)
    torch.cuda.synchronize()
    assert torch.equal(out, cu.out)


def test_lean_operator_without_scheduler_scratch_matches_full_operator():
    from mac_attention_b200 import make_decision_workspace

    ext = load_mac_persistent_decode_extension()
    case = synth.make_decode_case(batch=3, ctx=0, ctx_list=[2000, 3500, 900], hq=32, hkv=8,
                                  capacity=256, seed=14)
    synth.plant_matches(case, hit_fraction=0.5, borderline_fraction=0.5, seed=3)
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=128, front_sink_tokens=16)
    full = run_cuda(case, cfg)
    c = case.to("cuda").clone()
    dws = make_decision_workspace(3, 32, 8, 256, cfg.match_tile_slots)
    assert sum(t.numel() * t.element_size() for t in dws) < 1 << 20
    out = torch.empty_like(c.q_post)
    lse = torch.empty(3, 32, device="cuda")
    e = torch.empty(0)
    ext.mac_persistent_decode_bf16_lean(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids,
                                        c.past_lens, c.out_cache_loc, c.query_cache, c.attn_cache,
                                        c.lse_cache, out, lse, dws, *cfg.scalar_args(),
                                        c.query_cache, e, e, e)
    torch.cuda.synchronize()
    assert torch.equal(out, full.out) and torch.equal(lse, full.lse)
    for i, j in zip(range(16), range(16)):
        assert torch.equal(dws[i], full.ws[j])
    assert torch.equal(dws[16][:7], full.ws[22][:7])
    assert torch.equal(c.attn_cache, full.case.attn_cache)


def test_run_twice_is_bit_identical_and_graph_replay_matches():
    case = synth.make_decode_case(batch=4, ctx=2500, hq=32, hkv=8, capacity=512, seed=21)
    cfg = O.DecodeConfig(max_context=4096, bench_mode=1, bench_hit_rate=0.75, bench_seed=5)
    a = run_cuda(case, cfg)
    b = run_cuda(case, cfg)
    assert torch.equal(a.out, b.out) and torch.equal(a.lse, b.lse)
    assert torch.equal(a.case.attn_cache, b.case.attn_cache)
    # capture the same step into a CUDA graph (after the eager warm-up above) and replay
    ext = load_mac_persistent_decode_extension()
    c = case.to("cuda").clone()
    ws = make_decode_workspace(4, 32, 8, 512, 4096, 32, 32, 256)
    out = torch.zeros_like(c.q_post)
    lse = torch.zeros(4, 32, device="cuda")
    e = torch.empty(0)

    def launch():
        ext.mac_persistent_decode_bf16(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids,
                                       c.past_lens, c.out_cache_loc, c.query_cache, c.attn_cache,
                                       c.lse_cache, out, lse, *ws, *cfg.scalar_args(),
                                       c.query_cache, e, e, e)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        launch()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()
    out.zero_()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, a.out)
    _status_clean()


def test_step_tensors_in_pinned_host_memory_give_the_same_step():
    """q_post, q_pre and out may lie in pinned host memory (the kernel reads and writes them
    over the bus); a pageable host tensor is refused."""
    ext = load_mac_persistent_decode_extension()
    case = synth.make_decode_case(batch=3, ctx=0, ctx_list=[3000, 700, 1900], hq=32, hkv=8,
                                  capacity=256, seed=33)
    synth.plant_matches(case, hit_fraction=0.5, seed=4)
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=128, front_sink_tokens=16)
    want = run_cuda(case, cfg)
    c = case.to("cuda").clone()
    ws = make_decode_workspace(3, 32, 8, 256, 4096, 32, 32, 128, 16)
    lse = torch.empty(3, 32, device="cuda")
    e = torch.empty(0)
    q_post = case.q_post.cpu().pin_memory()
    q_pre = case.q_pre.cpu().pin_memory()
    out = torch.zeros(case.q_post.shape, dtype=torch.bfloat16).pin_memory()

    def call(q_post_t, q_pre_t, out_t):
        ext.mac_persistent_decode_bf16(q_post_t, q_pre_t, c.k, c.v, c.req_to_token, c.req_ids,
                                       c.past_lens, c.out_cache_loc, c.query_cache, c.attn_cache,
                                       c.lse_cache, out_t, lse, *ws, *cfg.scalar_args(),
                                       c.query_cache, e, e, e)

    call(q_post, q_pre, out)
    torch.cuda.synchronize()
    assert torch.equal(out, want.out.cpu()) and torch.equal(lse, want.lse)
    assert torch.equal(c.attn_cache, want.case.attn_cache)
    assert torch.equal(c.query_cache, want.case.query_cache)
    with pytest.raises(RuntimeError, match="pinned host memory"):
        call(q_post, q_pre, torch.zeros(case.q_post.shape, dtype=torch.bfloat16))
    _status_clean()


def test_hit_path_equals_full_attention_at_long_context():
    """Size-independent property at a full-size context: a step that reuses the
    prefix state written by the previous step gives the same output as exact
    full attention over the whole context with the same query."""
    ctx = 126976
    case = synth.make_decode_case(batch=2, ctx=ctx, hq=32, hkv=8, capacity=512, seed=3,
                                  kv_scale=1.0).to("cuda")
    cfg_miss = O.DecodeConfig(max_context=131072, gen_min_limit=1 << 30)
    cfg_hit = O.DecodeConfig(max_context=131072)
    r1 = run_cuda(case, cfg_miss)                      # writes ring rows for position ctx
    assert int(r1.ws[3].sum()) == 0
    step2 = r1.case.clone()
    step2.past_lens = step2.past_lens + 1
    # the next token reuses the pool row after the current one: extend the table
    r2t = torch.cat([step2.req_to_token, step2.req_to_token[:, -1:]], dim=1).contiguous()
    for n in range(2):
        r2t[n, ctx] = step2.out_cache_loc[n]
    step2.req_to_token = r2t
    # a fresh pool row for the new token: reuse the row of position 0 of the other request
    step2.out_cache_loc = torch.tensor([int(r2t[1, 7]), int(r2t[0, 7])], dtype=torch.int32,
                                       device="cuda")
    hit = run_cuda(step2, cfg_hit)
    full = run_cuda(step2, cfg_miss)
    assert int(hit.ws[3].sum()) == 2 * 32 and (hit.ws[5][:2] == ctx).all()
    assert int(hit.ws[22][5]) == 0 and int(full.ws[22][6]) == 16
    assert O.rel_l2(hit.out.float().cpu(), full.out.float().cpu()) < REL_L2_TOL
    assert (hit.lse - full.lse).abs().max() < 2e-2
    _status_clean()


def test_malformed_rows_are_zeroed_and_flagged():
    case = synth.make_decode_case(batch=3, ctx=400, hq=8, hkv=2, capacity=64, seed=2)
    case.req_ids = torch.tensor([0, 99, 2], dtype=torch.int32)     # 99 is outside the ring
    cfg = O.DecodeConfig(max_context=512, semantic_pos_ahead=16)
    cu = run_cuda(case, cfg)
    orc, _ = run_oracle(case, cfg)
    assert orc.bad_rows == 1
    assert torch.equal(cu.out[1], torch.zeros_like(cu.out[1]))
    assert O.rel_l2(cu.out.float().cpu(), orc.out_f32) < REL_L2_TOL
    assert ops.query_status() & 0x2
    assert ops.query_status() == 0  # reading clears it


def test_bounded_wait_gives_up_and_reports_without_hanging():
    """A wait that nothing completes runs out after its limit, the kernel
    returns, the status word says so, and the next decode step works."""
    status, gave_up = ops.selftest_bounded_wait()
    assert gave_up == 2
    assert status & 0x1
    assert ops.query_status() == 0
    case = synth.make_decode_case(batch=2, ctx=600, hq=8, hkv=2, capacity=64, seed=3)
    cfg = O.DecodeConfig(max_context=1024, semantic_pos_ahead=16)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_outputs_close(cu, orc, orc_case)
    _status_clean()


def test_scratch_growth_is_refused_during_graph_capture():
    ext = load_mac_persistent_decode_extension()
    cfg = O.DecodeConfig(max_context=256, semantic_pos_ahead=16)
    # far more KV groups than any other test: the scratch arena has to grow
    if ops.launch_info()["arena_bytes"] > (45 << 20):
        pytest.skip("the scratch arena is already large enough for this shape")
    case = synth.make_decode_case(batch=500, ctx=40, hq=64, hkv=8, capacity=8, seed=1).to("cuda")
    ws = make_decode_workspace(500, 64, 8, 8, 256, 32, 32, 16)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(500, 64, device="cuda")
    e = torch.empty(0)

    def launch():
        ext.mac_persistent_decode_bf16(case.q_post, case.q_pre, case.k, case.v, case.req_to_token,
                                       case.req_ids, case.past_lens, case.out_cache_loc,
                                       case.query_cache, case.attn_cache, case.lse_cache, out, lse,
                                       *ws, *cfg.scalar_args(), case.query_cache, e, e, e)

    graph = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="captured"):
        with torch.cuda.graph(graph):
            launch()
    torch.cuda.synchronize()
    launch()                      # eager call grows the arena ...
    torch.cuda.synchronize()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):  # ... after which capture works
        launch()
    graph2.replay()
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    _status_clean()


def test_argument_errors_raise_like_the_reference():
    ext = load_mac_persistent_decode_extension()
    case = synth.make_decode_case(batch=1, ctx=100, hq=8, hkv=2, capacity=16, seed=1).to("cuda")
    cfg = O.DecodeConfig(max_context=128, semantic_pos_ahead=8)
    ws = make_decode_workspace(1, 8, 2, 16, 128, 32, 32, 8)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(1, 8, device="cuda")
    e = torch.empty(0)

    def call(**over):
        a = dict(q_post=case.q_post, q_pre=case.q_pre, k=case.k, out=out, scal=cfg.scalar_args(),
                 ws=ws)
        a.update(over)
        ext.mac_persistent_decode_bf16(a["q_post"], a["q_pre"], a["k"], case.v, case.req_to_token,
                                       case.req_ids, case.past_lens, case.out_cache_loc,
                                       case.query_cache, case.attn_cache, case.lse_cache, a["out"],
                                       lse, *a["ws"], *a["scal"], case.query_cache, e, e, e)

    with pytest.raises(RuntimeError, match="wrong dtype"):
        call(q_post=case.q_post.float())
    with pytest.raises(RuntimeError, match="must be CUDA"):
        call(q_pre=case.q_pre.cpu())
    with pytest.raises(RuntimeError, match="shape mismatch"):
        call(out=torch.empty(1, 8, 64, device="cuda", dtype=torch.bfloat16))
    bad_scal = list(cfg.scalar_args())
    bad_scal[11] = 5
    with pytest.raises(RuntimeError, match="bench mode"):
        call(scal=bad_scal)
    small_ws = make_decode_workspace(1, 8, 2, 16, 64, 32, 32, 8)
    with pytest.raises(RuntimeError, match="rect workspace too small"):
        call(ws=small_ws)
    call()
    torch.cuda.synchronize()


def _reference_decode():
    from oracle import build_ref

    try:
        return build_ref.load_decode()
    except Exception:  # noqa: BLE001
        return None


def test_decisions_identical_to_reference_cuda_kernel():
    """The reference's own kernel (compiled for sm_100a from its source file) and
    this kernel on the same device tensors: decision arrays bit-identical,
    outputs within the stated tolerance of each other."""
    ref = _reference_decode()
    if ref is None:
        pytest.skip("reference kernel was not built for this box (oracle/_ref missing)")
    torch.manual_seed(0)
    for spec in CASES[:3]:
        case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"],
                                      hq=spec["hq"], hkv=spec["hkv"], capacity=spec["capacity"],
                                      page_size=spec["page"], seed=77)
        synth.plant_matches(case, hit_fraction=0.5, noise=0.1, borderline_fraction=0.6, seed=6)
        cfg = O.DecodeConfig(max_context=8192, semantic_pos_ahead=spec["S"],
                             front_sink_tokens=spec["F"], match_tile_slots=spec["mts"])
        mine = run_cuda(case, cfg)
        theirs = run_cuda(case, cfg, ext=ref, poison=False)
        for idx in (3, 4, 5, 6, 7, 8, 9, 15):
            assert torch.equal(mine.ws[idx], theirs.ws[idx]), f"workspace[{idx}] differs"
        assert int(mine.ws[22][5]) == int(theirs.ws[22][5])
        assert int(mine.ws[22][6]) == int(theirs.ws[22][6])
        assert O.rel_l2(mine.out.float().cpu(), theirs.out.float().cpu()) < 2 * REL_L2_TOL
        assert torch.equal(mine.case.query_cache, theirs.case.query_cache)
        assert O.rel_l2(mine.case.attn_cache.float().cpu(), theirs.case.attn_cache.float().cpu()) < 2 * REL_L2_TOL
    # synthetic decisions, including the float rounding edge 0.1 * 5 + 0.5
    case = synth.make_decode_case(batch=5, ctx=2000, hq=8, hkv=1, capacity=512, seed=5)
    for mode, rate in ((2, 0.9), (1, 0.9), (1, 0.5)):
        cfg = O.DecodeConfig(max_context=4096, bench_mode=mode, bench_hit_rate=rate, bench_seed=7)
        mine = run_cuda(case, cfg)
        theirs = run_cuda(case, cfg, ext=ref, poison=False)
        for idx in (3, 4, 5, 6, 7, 8, 9, 15):
            assert torch.equal(mine.ws[idx], theirs.ws[idx]), f"bench workspace[{idx}] differs"


def test_decisions_at_serving_size_match_the_oracle():
    """16 requests at context 126976 with a 2048-slot ring (the benchmark's geometry, a
    quarter of its batch): planted matches per KV group plus rows within 1 % of the
    threshold on either side.  The K/V pool (8.6 GB) stays on the GPU; the CPU oracle
    restates the decisions alone from the ring and the queries."""
    batch, ctx, hq, hkv, M = 16, 126976, 32, 8, 2048
    case = synth.make_decode_case(batch=batch, ctx=ctx, hq=hq, hkv=hkv, capacity=M, page_size=16,
                                  seed=12, device="cuda")
    planted = synth.plant_matches(case, hit_fraction=0.7, noise=0.1, borderline_fraction=0.6,
                                  seed=4, lag_lo=1, lag_hi=M, heads_per_draw=hq // hkv)
    cfg = O.DecodeConfig(max_context=131072)
    ext = load_mac_persistent_decode_extension()
    ws = make_decode_workspace(batch, hq, hkv, M, cfg.max_context, cfg.tile_tokens,
                               cfg.match_tile_slots, cfg.semantic_pos_ahead, 0)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(batch, hq, device="cuda")
    ring_before = case.query_cache.cpu()
    lse_before = case.lse_cache.cpu()
    e = torch.empty(0)
    ext.mac_persistent_decode_bf16(case.q_post, case.q_pre, case.k, case.v, case.req_to_token,
                                   case.req_ids, case.past_lens, case.out_cache_loc,
                                   case.query_cache, case.attn_cache, case.lse_cache, out, lse, *ws,
                                   *cfg.scalar_args(), case.query_cache, e, e, e)
    torch.cuda.synchronize()
    hit, mslot, mpos = O.decide(case.q_pre.cpu(), case.req_ids.cpu(), case.past_lens.cpu(),
                                ring_before, lse_before, cfg, hkv=hkv,
                                req_to_token_shape=tuple(case.req_to_token.shape))
    got_hit = ws[3][:batch].cpu()
    assert torch.equal(got_hit, hit)
    sel = hit.bool()
    assert torch.equal(ws[4][:batch].cpu()[sel], mslot[sel])
    assert torch.equal(ws[5][:batch].cpu()[sel], mpos[sel])
    assert planted.sum() > 0 and bool((got_hit.bool() | ~planted).all())   # every planted head hits
    assert int(got_hit.sum()) > int(planted.sum())                         # and some borderline rows do
    assert torch.isfinite(out.float()).all()
    _status_clean()


@pytest.mark.parametrize("hq,hkv", [(16, 2), (8, 2), (8, 8)], ids=["gqa8", "gqa4", "mha"])
def test_long_context_few_groups_outputs_match_oracle(hq, hkv):
    """Two requests with tens of thousands of tokens and only a handful of KV groups: every
    full-attention group is cut into dozens of pieces, so its partials take the staged
    (shared-memory) merge.  Outputs, ring rows and LSEs against the CPU oracle."""
    case = synth.make_decode_case(batch=2, ctx=0, ctx_list=[40000, 23000], hq=hq, hkv=hkv,
                                  capacity=256, page_size=16, seed=21)
    synth.plant_matches(case, hit_fraction=0.4, noise=0.1, seed=8, lag_hi=200,
                        heads_per_draw=hq // hkv)
    cfg = O.DecodeConfig(max_context=65536, semantic_pos_ahead=256)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 2)
    assert_outputs_close(cu, orc, orc_case)
    assert int(cu.ws[22][0]) >= 40          # pieces: far more than groups
    assert 0 < int(orc.head_hit.sum()) < orc.head_hit.numel()
    _status_clean()


def test_overlapping_launch_on_another_stream_is_refused():
    """Decode launches of one device share scratch and barrier words.  A second launch on
    another stream while the first is still running must be refused with a clear error, not
    left to race; after the first has finished the same call goes through."""
    case = synth.make_decode_case(batch=8, ctx=60000, hq=32, hkv=8, capacity=256, page_size=16,
                                  seed=3, device="cuda")
    cfg = O.DecodeConfig(max_context=65536, gen_min_limit=10 ** 6)      # every group: full attention
    ext = load_mac_persistent_decode_extension()
    ws = make_decode_workspace(8, 32, 8, 256, cfg.max_context, cfg.tile_tokens,
                               cfg.match_tile_slots, cfg.semantic_pos_ahead, 0,
                               partial_dtype=torch.bfloat16)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(8, 32, device="cuda")
    e = torch.empty(0)

    def call():
        ext.mac_persistent_decode_bf16(case.q_post, case.q_pre, case.k, case.v, case.req_to_token,
                                       case.req_ids, case.past_lens, case.out_cache_loc,
                                       case.query_cache, case.attn_cache, case.lse_cache, out, lse,
                                       *ws, *cfg.scalar_args(), case.query_cache, e, e, e)

    call()
    torch.cuda.synchronize()
    want = out.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for _ in range(4):          # a few steps queued back to back keep the device busy
        call()
    with torch.cuda.stream(side):
        with pytest.raises(RuntimeError, match="another stream"):
            call()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        call()                  # nothing in flight any more: accepted
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    _status_clean()

