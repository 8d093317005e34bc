"""The match-scan variants of the decode kernel must be indistinguishable: per-thread
cp.async staging with a 128-byte probe (the default) and bulk tensor copies with a 64- or
128-byte probe (``MAC_B200_SCAN`` = ``cpasync`` / ``bulk64`` / ``bulk128``, read at every
launch).  Each runs a seeded slice of the random parity
matrix against the CPU oracle -- including head counts that do not divide the
256-row copy box (G = 3, 5, 7), 128 query heads, rings shorter than a box and
contexts shorter than the ring -- and all of them must report bit-identical
per-tile match arrays below the threshold and identical decision arrays.
"""
import random

import pytest
import torch

from mac_attention_b200 import ops, synth
from oracle import mac_oracle as O

from helpers import assert_decisions_equal, assert_outputs_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu

MODES = ["cpasync", "bulk64", "bulk128"]


@pytest.fixture
def scan_mode(monkeypatch):
    def set_mode(mode):
        monkeypatch.setenv("MAC_B200_SCAN", mode)
    return set_mode


def _draw(rng):
    hkv = rng.choice([1, 2, 4, 8, 16])
    g = rng.choice([1, 2, 3, 4, 5, 7, 8])
    batch = rng.randint(1, 4)
    capacity = rng.choice([5, 8, 64, 200, 256, 512, 1024])
    ctxs = [rng.choice([rng.randint(1, 40), rng.randint(40, 900), rng.randint(900, 2500)])
            for _ in range(batch)]
    return dict(batch=batch, hq=hkv * g, hkv=hkv, capacity=capacity, ctxs=ctxs,
                S=rng.choice([1, 16, 64, 256]), F=rng.choice([0, 0, 16, 64]),
                mts=rng.choice([8, 24, 32, 64]), threshold=rng.choice([0.3, 0.45, 0.6]),
                cand=rng.choice([(0, 0), (0, 0), (7, 1)]), gen_min=rng.choice([0, 0, 500]),
                gate=rng.random() < 0.25, hit=rng.choice([0.0, 0.4, 0.8, 1.0]),
                borderline=rng.choice([0.0, 0.6]), seed=rng.randint(0, 10 ** 6))


def _case(spec):
    case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"], hq=spec["hq"],
                                  hkv=spec["hkv"], capacity=spec["capacity"], page_size=16,
                                  seed=spec["seed"])
    synth.plant_matches(case, hit_fraction=spec["hit"], noise=0.1,
                        borderline_fraction=spec["borderline"], seed=spec["seed"] + 1,
                        lag_hi=spec["capacity"], threshold=spec["threshold"])
    if spec["gate"]:
        synth.add_readiness_gate(case, not_ready_fraction=0.3, stale_fraction=0.2,
                                 seed=spec["seed"] + 2)
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=spec["S"],
                         front_sink_tokens=spec["F"], match_tile_slots=spec["mts"],
                         threshold=spec["threshold"], gen_min_limit=spec["gen_min"],
                         lookback_right=spec["cand"][0], candidate_mode=spec["cand"][1])
    return case, cfg


@pytest.mark.parametrize("chunk", range(8))
def test_scan_variants_agree_with_the_oracle_and_with_each_other(chunk, scan_mode):
    rng = random.Random(31000 + chunk)
    for i in range(12):
        spec = _draw(rng)
        case, cfg = _case(spec)
        orc, orc_case = run_oracle(case, cfg)
        thr = O.threshold_distance(spec["threshold"])
        below = orc.match_dist < thr
        runs = {}
        for mode in MODES:
            scan_mode(mode)
            cu = run_cuda(case, cfg)
            tag = f"mode {mode} chunk {chunk} case {i}: {spec}"
            try:
                assert_decisions_equal(cu, orc, spec["batch"])
                assert_outputs_close(cu, orc, orc_case)
            except AssertionError as exc:
                raise AssertionError(f"{tag}\n{exc}") from exc
            md, mp, ms = (cu.ws[j][:spec["batch"]].cpu() for j in (0, 1, 2))
            assert torch.equal(md[below], orc.match_dist[below]), tag
            assert torch.equal(mp[below], orc.match_pos[below]), tag
            assert torch.equal(ms[below], orc.match_slot[below]), tag
            assert ops.query_status() == 0, tag
            runs[mode] = cu
        for mode in MODES[1:]:
            for idx in (3, 4, 5, 6, 7, 8, 9, 15):
                assert torch.equal(runs[mode].ws[idx], runs[MODES[0]].ws[idx]), (mode, idx, spec)
            assert torch.equal(runs[mode].case.query_cache, runs[MODES[0]].case.query_cache)


@pytest.mark.parametrize("mode", MODES)
def test_rows_whose_distance_hides_in_the_unprobed_dims(mode, scan_mode):
    """Ring rows that are identical to the query on the probed prefix and far on the rest
    (the probe sees distance 0) and rows that are far on the prefix only: the first kind
    must reach the exact evaluation and be rejected there, the second kind may be dropped
    by the probe; neither can change a decision."""
    scan_mode(mode)
    case = synth.make_decode_case(batch=2, ctx=0, ctx_list=[1500, 700], hq=16, hkv=4, capacity=256,
                                  page_size=16, seed=5)
    g = torch.Generator().manual_seed(3)
    for n in range(2):
        P, req = int(case.past_lens[n]), int(case.req_ids[n])
        for h in range(16):
            q = case.q_pre[n, h].float()
            for j, split in enumerate((32, 64, 96)):
                row = q.clone()
                row[split:] += 3.0 * torch.randn(128 - split, generator=g)     # far beyond the prefix
                case.query_cache[req, (P - 3 - j) % 256, h] = row.to(torch.bfloat16)
                row = q.clone()
                row[:split] += 3.0 * torch.randn(split, generator=g)           # far on the prefix
                case.query_cache[req, (P - 9 - j) % 256, h] = row.to(torch.bfloat16)
            if h % 3 == 0:    # and a true near-duplicate further back
                case.query_cache[req, (P - 40) % 256, h] = (q + 0.05 * torch.randn(128, generator=g)).to(torch.bfloat16)
                case.lse_cache[req, (P - 40) % 256, h] = 4.0
    cfg = O.DecodeConfig(max_context=4096, semantic_pos_ahead=64)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 2)
    assert_outputs_close(cu, orc, orc_case)
    assert 0 < int(orc.head_hit.sum()) < orc.head_hit.numel()
    assert ops.query_status() == 0


@pytest.mark.parametrize("knobs", [
    {"MAC_B200_PIECE_WAVES": "2"}, {"MAC_B200_PIECE_WAVES": "4"},
    {"MAC_PERSISTENT_COOP_CTAS": "37"}, {"MAC_PERSISTENT_COOP_CTAS": "5", "MAC_B200_PIECE_WAVES": "4"},
    {"MAC_B200_MIN_PIECE": "64", "MAC_B200_FUSE_MAX": "0"}, {"MAC_B200_OVH_TOK": "64"},
], ids=lambda k: "_".join(f"{a[9:]}{b}" for a, b in k.items()))
def test_schedule_knobs_do_not_change_results(knobs, monkeypatch):
    """The attention schedule's tuning knobs (pieces per CTA, a capped grid, the smallest piece,
    no fused groups, the row-opening cost) only move work between CTAs: with several pieces per
    CTA the later ones are pulled through the ticket, with a capped grid one CTA walks many
    groups.  Decisions and outputs stay those of the oracle."""
    for name, value in knobs.items():
        monkeypatch.setenv(name, value)
    rng = random.Random(77)
    for i in range(6):
        spec = _draw(rng)
        spec["ctxs"] = [rng.choice([rng.randint(2000, 9000), rng.randint(300, 900)]) for _ in spec["ctxs"]]
        case, cfg = _case(spec)
        cfg.max_context = 16384
        orc, orc_case = run_oracle(case, cfg)
        cu = run_cuda(case, cfg)
        tag = f"{knobs} case {i}: {spec}"
        try:
            assert_decisions_equal(cu, orc, spec["batch"])
            assert_outputs_close(cu, orc, orc_case)
        except AssertionError as exc:
            raise AssertionError(f"{tag}\n{exc}") from exc
        assert ops.query_status() == 0, tag
