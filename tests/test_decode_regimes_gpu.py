"""Output parity against the CPU oracle in the numerical regimes the benchmark
times (the BASELINE configurations at or near their full context lengths):

* GQA-8 with front-sink tokens and sink-heavy softmax mass (keys of the first 64
  positions scaled x4) at context 65536;
* the Llama-70B attention shape (Hq 64 / Hkv 8) at context 65536, and one
  KV-head shard of it (Hq 8 / Hkv 1) at the full 126976;
* a ragged mixed serving step: contexts drawn from [8K, 127K], 30 % of the
  requests gated off (not ready or stale epoch), the rest hitting at 0.8;
* the headline geometry itself (GQA-4, context 126976, ring 2048) on a few
  requests with the synthetic-decision mode the benchmark uses.

Cases are generated on the GPU and copied to the host for the oracle; decisions
must be equal, outputs and ring states within 1e-2 relative L2, LSEs within
2e-2 (tolerances in ``tests/helpers.py``).
"""
import pytest
import torch

from mac_attention_b200 import ops, synth
from oracle import mac_oracle as O
from tests.helpers import assert_decisions_equal, assert_outputs_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


def _check(case, cfg, n, expect_hits=True, expect_misses=True):
    cu = run_cuda(case, cfg, partial_dtype=torch.bfloat16)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, n)
    assert_outputs_close(cu, orc, orc_case)
    hits = int(orc.head_hit.sum())
    if expect_hits:
        assert hits > 0
    if expect_misses:
        assert hits < orc.head_hit.numel()
    assert ops.query_status() == 0
    return cu, orc


@pytest.mark.parametrize("front_sink", [64, 128])
@pytest.mark.parametrize("hit", [0.5, 0.9])
def test_gqa8_sink_heavy_softmax_at_64k(front_sink, hit):
    """BASELINE config 2: Hq 32 / Hkv 4, context 65536, F in {64, 128}, the first 64 keys
    scaled x4 so that most of the softmax mass sits on the sink tokens."""
    n = 3
    case = synth.make_decode_case(batch=n, ctx=65536, hq=32, hkv=4, capacity=2048, page_size=16,
                                  seed=31 + front_sink, device="cuda", sink_boost=64)
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, front_sink_tokens=front_sink,
                         bench_mode=1, bench_hit_rate=hit, bench_match_lag_mean=64.0, bench_seed=1)
    _check(case, cfg, n)


def test_gqa8_sink_heavy_real_scan_with_planted_rows():
    """Same regime with decisions from the real match scan (planted ring rows per KV group)."""
    n = 2
    case = synth.make_decode_case(batch=n, ctx=65536, hq=32, hkv=4, capacity=2048, page_size=16,
                                  seed=77, device="cuda", sink_boost=64)
    synth.plant_matches(case, hit_fraction=0.6, noise=0.1, borderline_fraction=0.5, seed=6,
                        lag_lo=1, lag_hi=1500, heads_per_draw=8)
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, front_sink_tokens=64)
    _check(case, cfg, n)


def test_llama70b_shape_at_64k():
    """BASELINE config 3 shape, unsplit: Hq 64 / Hkv 8, four requests at context 65536."""
    n = 4
    case = synth.make_decode_case(batch=n, ctx=65536, hq=64, hkv=8, capacity=2048, page_size=16,
                                  seed=41, device="cuda")
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, bench_mode=1,
                         bench_hit_rate=0.9, bench_match_lag_mean=64.0, bench_seed=1)
    _check(case, cfg, n)


def test_llama70b_kv_head_shard_at_full_context():
    """One KV-head shard of config 3 as an 8-GPU split sees it: Hq 8 / Hkv 1, context 126976."""
    n = 6
    case = synth.make_decode_case(batch=n, ctx=126976, hq=8, hkv=1, capacity=2048, page_size=16,
                                  seed=43, device="cuda")
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, bench_mode=1,
                         bench_hit_rate=0.7, bench_match_lag_mean=64.0, bench_seed=1)
    _check(case, cfg, n)


def test_ragged_mixed_serving_step_with_gated_requests():
    """BASELINE config 4: eight GQA-4 requests with contexts drawn from [8K, 127K], 30 % of
    them gated off (not ready, or a stale cache epoch) and demoted to full attention in the
    launch; the rest hit at 0.8."""
    n = 8
    g = torch.Generator().manual_seed(4)
    ctxs = torch.randint(8192, 126977, (n,), generator=g).tolist()
    case = synth.make_decode_case(batch=n, ctx=0, ctx_list=ctxs, hq=32, hkv=8, capacity=2048,
                                  page_size=16, seed=44, device="cuda")
    synth.add_readiness_gate(case, not_ready_fraction=0.2, stale_fraction=0.1, seed=4)
    off = case.meta["gated_off"]
    if not bool(off.any()):          # the draw must gate at least two requests
        off[:2] = True
        case.cache_ready[:2] = False
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, bench_mode=1,
                         bench_hit_rate=0.8, bench_match_lag_mean=64.0, bench_seed=1)
    before = case.clone()
    cu, orc = _check(case, cfg, n)
    after = cu.case
    for i in range(n):
        req = int(case.req_ids[i])
        if bool(off[req]):
            assert int(cu.ws[3][i].sum()) == 0 and bool((cu.ws[15][i] == 1).all())
            assert torch.equal(after.query_cache[req], before.query_cache[req])
            assert torch.equal(after.lse_cache[req], before.lse_cache[req])


def test_ragged_mixed_step_real_scan():
    """Config-4 geometry with planted matches and the real scan (no synthetic override)."""
    n = 5
    ctxs = [9000, 100000, 33333, 126976, 61000]
    case = synth.make_decode_case(batch=n, ctx=0, ctx_list=ctxs, hq=32, hkv=8, capacity=2048,
                                  page_size=16, seed=45, device="cuda")
    synth.plant_matches(case, hit_fraction=0.8, noise=0.1, borderline_fraction=0.4, seed=9,
                        lag_lo=1, lag_hi=2048, heads_per_draw=4)
    synth.add_readiness_gate(case, not_ready_fraction=0.2, stale_fraction=0.2, seed=11)
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256)
    _check(case, cfg, n)


@pytest.mark.parametrize("hit", [0.0, 0.75, 1.0])
def test_headline_geometry_outputs(hit):
    """The benchmark's own geometry (GQA-4, context 126976, ring 2048, synthetic decisions,
    lag 64) on six requests: outputs, ring rows and LSEs against the oracle."""
    n = 6
    case = synth.make_decode_case(batch=n, ctx=126976, hq=32, hkv=8, capacity=2048, page_size=16,
                                  seed=1000, device="cuda")
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, bench_mode=1,
                         bench_hit_rate=hit, bench_match_lag_mean=64.0, bench_seed=1)
    _check(case, cfg, n, expect_hits=hit > 0, expect_misses=hit < 1)


def test_matched_prefix_anywhere_in_the_context_extension(monkeypatch):
    """The labelled benchmark extension (``MAC_B200_BENCH_LONG_BAND=1``): with synthetic
    decisions a reused entry may lie anywhere in the context (BASELINE config 1 draws the
    matched prefix from [50 %, 95 %] of it), i.e. the band a hit head recomputes is tens of
    thousands of tokens long.  Decisions and outputs against the oracle with the same switch;
    with the switch off (the default) the same step demotes those heads like the reference."""
    n = 3
    case = synth.make_decode_case(batch=n, ctx=60000, hq=32, hkv=8, capacity=2048, page_size=16,
                                  seed=61, device="cuda")
    cfg = O.DecodeConfig(max_context=131072, semantic_pos_ahead=256, bench_mode=1,
                         bench_hit_rate=0.75, bench_skip_ratio=0.725, bench_skip_ratio_std=0.13,
                         bench_seed=1, bench_long_band=1)
    monkeypatch.setenv("MAC_B200_BENCH_LONG_BAND", "1")
    cu, orc = _check(case, cfg, n)
    hit = orc.head_hit.bool()
    band = (orc.head_new_end - orc.head_rect_start)[hit]
    assert int(band.max()) > 2048 * 4          # far beyond the ring's span
    monkeypatch.delenv("MAC_B200_BENCH_LONG_BAND")
    cfg.bench_long_band = 0
    cu2 = run_cuda(case, cfg, partial_dtype=torch.bfloat16)
    orc2, _ = run_oracle(case, cfg)
    assert_decisions_equal(cu2, orc2, n)
    hit2 = orc2.head_hit.bool()
    band2 = (orc2.head_new_end - orc2.head_rect_start)[hit2]
    assert band2.numel() == 0 or int(band2.max()) <= 2048
    assert int(hit2.sum()) < int(hit.sum())
