"""Randomised parity matrix of the decode step: 860 seeded small cases over
the whole argument space (GQA shapes, ragged contexts shorter and longer than the
ring, window and sink sizes, page sizes, match-tile sizes, thresholds, candidate
modes, readiness gates, synthetic-decision modes), each one compared with the CPU
oracle: decisions identical, outputs / ring rows / LSEs within 1e-2 relative L2.

The reference states such a matrix ("identical match/hit decisions, 1e-2 relative
L2", README.md:96-99 of the reference project) without shipping the harness."""
import os
import random

import pytest
import torch

from mac_attention_b200 import ops, synth
from oracle import mac_oracle as O

from helpers import assert_decisions_equal, assert_outputs_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu

CHUNKS, PER_CHUNK = 43, 20   # 860 cases
SEED_BASE = int(os.environ.get("MAC_MATRIX_SEED", "0"))   # another base draws another 860


def _draw(rng: random.Random):
    hkv = rng.choice([1, 2, 4, 8])
    g = rng.choice([1, 2, 4, 8])
    batch = rng.randint(1, 5)
    capacity = rng.choice([8, 16, 64, 200, 256, 512])
    S = rng.choice([1, 4, 16, 64, 256])
    F = rng.choice([0, 0, 4, 16, 64, 128])
    ctxs = [rng.choice([rng.randint(1, 40), rng.randint(40, 700), rng.randint(700, 1500)])
            for _ in range(batch)]
    spec = dict(
        batch=batch, hq=hkv * g, hkv=hkv, capacity=capacity, S=S, F=F, ctxs=ctxs,
        page=rng.choice([1, 8, 16]), mts=rng.choice([8, 24, 32]),
        threshold=rng.choice([0.3, 0.45, 0.45, 0.6]),
        gen_min=rng.choice([0, 0, 0, 300]),
        cand=rng.choice([(0, 0), (0, 0), (5, 1)]),          # (lookback_right, candidate_mode)
        gate=rng.random() < 0.25,
        bench=rng.choice([0, 0, 0, 1, 2]),
        hit=rng.choice([0.0, 0.3, 0.6, 0.9, 1.0]),
        borderline=rng.choice([0.0, 0.5]),
        seed=rng.randint(0, 10 ** 6),
    )
    return spec


@pytest.mark.parametrize("chunk", range(CHUNKS))
def test_randomised_parity_matrix(chunk):
    rng = random.Random(1000 + chunk + 100000 * SEED_BASE)
    for i in range(PER_CHUNK):
        spec = _draw(rng)
        case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"],
                                      hq=spec["hq"], hkv=spec["hkv"], capacity=spec["capacity"],
                                      page_size=spec["page"], seed=spec["seed"])
        synth.plant_matches(case, hit_fraction=spec["hit"], noise=0.1,
                            borderline_fraction=spec["borderline"], seed=spec["seed"] + 1,
                            lag_hi=spec["capacity"], threshold=spec["threshold"])
        if spec["gate"]:
            synth.add_readiness_gate(case, not_ready_fraction=0.3, stale_fraction=0.2,
                                     seed=spec["seed"] + 2)
        cfg = O.DecodeConfig(max_context=2048, semantic_pos_ahead=spec["S"],
                             front_sink_tokens=spec["F"], match_tile_slots=spec["mts"],
                             threshold=spec["threshold"], gen_min_limit=spec["gen_min"],
                             lookback_right=spec["cand"][0], candidate_mode=spec["cand"][1],
                             bench_mode=spec["bench"], bench_hit_rate=spec["hit"],
                             bench_match_lag_mean=float(min(64, spec["capacity"])),
                             bench_seed=spec["seed"] % 97)
        tag = f"chunk {chunk} case {i}: {spec}"
        try:
            cu = run_cuda(case, cfg)
            orc, orc_case = run_oracle(case, cfg)
            assert_decisions_equal(cu, orc, spec["batch"])
            assert_outputs_close(cu, orc, orc_case)
        except AssertionError as exc:
            raise AssertionError(f"{tag}\n{exc}") from exc
        assert ops.query_status() == 0, tag


def _draw_reference_range(rng: random.Random):
    """The same draw, kept inside the parameter ranges the reference's own tests,
    checker and benchmarks exercise (match tile 32, window >= 16, ring >= 64)."""
    spec = _draw(rng)
    spec["mts"] = 32
    spec["S"] = rng.choice([16, 64, 256])
    spec["capacity"] = rng.choice([64, 256, 512])
    spec["cand"] = (0, 0)
    spec["gen_min"] = 0
    return spec


@pytest.mark.parametrize("chunk", range(5))
def test_randomised_matrix_against_the_reference_kernel(chunk):
    """100 of the random cases through the reference's own CUDA kernel (built for
    sm_100a from its source file): decision arrays bit-identical, outputs and ring
    rows within twice the stated tolerance of each other."""
    from oracle import build_ref

    try:
        ref = build_ref.load_decode()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is None:
        pytest.skip("reference kernel was not built for this box")
    rng = random.Random(5000 + chunk)
    for i in range(PER_CHUNK):
        spec = _draw_reference_range(rng)
        case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"],
                                      hq=spec["hq"], hkv=spec["hkv"], capacity=spec["capacity"],
                                      page_size=spec["page"], seed=spec["seed"])
        synth.plant_matches(case, hit_fraction=spec["hit"], noise=0.1,
                            borderline_fraction=spec["borderline"], seed=spec["seed"] + 1,
                            lag_hi=spec["capacity"], threshold=spec["threshold"])
        if spec["gate"]:
            synth.add_readiness_gate(case, not_ready_fraction=0.3, stale_fraction=0.2,
                                     seed=spec["seed"] + 2)
        cfg = O.DecodeConfig(max_context=2048, semantic_pos_ahead=spec["S"],
                             front_sink_tokens=spec["F"], match_tile_slots=32,
                             threshold=spec["threshold"], bench_mode=spec["bench"],
                             bench_hit_rate=spec["hit"],
                             bench_match_lag_mean=float(min(64, spec["capacity"])),
                             bench_seed=spec["seed"] % 97)
        tag = f"chunk {chunk} case {i}: {spec}"
        mine = run_cuda(case, cfg)
        theirs = run_cuda(case, cfg, ext=ref, poison=False)
        for idx in (3, 4, 5, 6, 7, 8, 9, 15):
            assert torch.equal(mine.ws[idx], theirs.ws[idx]), f"workspace[{idx}] differs, {tag}"
        fin = torch.isfinite(theirs.lse)
        assert torch.equal(torch.isfinite(mine.lse), fin), tag
        assert O.rel_l2(mine.out.float().cpu(), theirs.out.float().cpu()) < 2e-2, tag
        assert torch.equal(mine.case.query_cache, theirs.case.query_cache), tag
        a, b = mine.case.attn_cache.float().cpu(), theirs.case.attn_cache.float().cpu()
        assert O.rel_l2(a, b) < 2e-2, tag


@pytest.mark.parametrize("F", [0, 16])
def test_zero_window_is_handled(F):
    """S = 0 (no trailing window: the ring row covers the whole context, current token
    included) is not exercised anywhere in the reference, whose band producer would read
    req_to_token[P]; here the current token always comes from out_cache_loc."""
    rng = random.Random(77 + F)
    for i in range(12):
        spec = _draw(rng)
        case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"],
                                      hq=spec["hq"], hkv=spec["hkv"], capacity=spec["capacity"],
                                      page_size=spec["page"], seed=spec["seed"])
        # the slot a real request has not filled yet: a wild pool row, so that reading it shows
        for n in range(spec["batch"]):
            case.req_to_token[int(case.req_ids[n]), int(case.past_lens[n])] = 0
        synth.plant_matches(case, hit_fraction=0.6, noise=0.1, seed=spec["seed"] + 1,
                            lag_hi=spec["capacity"])
        cfg = O.DecodeConfig(max_context=2048, semantic_pos_ahead=0, front_sink_tokens=F,
                             match_tile_slots=spec["mts"])
        cu = run_cuda(case, cfg)
        orc, orc_case = run_oracle(case, cfg)
        assert_decisions_equal(cu, orc, spec["batch"])
        assert_outputs_close(cu, orc, orc_case)
        assert ops.query_status() == 0


@pytest.mark.parametrize("chunk", range(3))
def test_randomised_parity_matrix_medium_contexts(chunk):
    """Contexts of thousands to tens of thousands of tokens on one to four requests: rows
    are cut into many pieces, so split-KV partials, the direct and the staged group merge,
    fused small groups and mixed groups all meet in one step."""
    rng = random.Random(9000 + chunk + 100000 * SEED_BASE)
    for i in range(10):
        spec = _draw(rng)
        spec["batch"] = rng.randint(1, 4)
        spec["ctxs"] = [rng.choice([rng.randint(3000, 9000), rng.randint(9000, 40000), rng.randint(50, 900)])
                        for _ in range(spec["batch"])]
        spec["capacity"] = rng.choice([64, 256, 512])
        case = synth.make_decode_case(batch=spec["batch"], ctx=0, ctx_list=spec["ctxs"],
                                      hq=spec["hq"], hkv=spec["hkv"], capacity=spec["capacity"],
                                      page_size=spec["page"], seed=spec["seed"])
        synth.plant_matches(case, hit_fraction=spec["hit"], noise=0.1,
                            borderline_fraction=spec["borderline"], seed=spec["seed"] + 1,
                            lag_hi=spec["capacity"], threshold=spec["threshold"])
        if spec["gate"]:
            synth.add_readiness_gate(case, not_ready_fraction=0.3, stale_fraction=0.2,
                                     seed=spec["seed"] + 2)
        cfg = O.DecodeConfig(max_context=65536, semantic_pos_ahead=spec["S"],
                             front_sink_tokens=spec["F"], match_tile_slots=spec["mts"],
                             threshold=spec["threshold"], bench_mode=spec["bench"],
                             bench_hit_rate=spec["hit"],
                             bench_match_lag_mean=float(min(64, spec["capacity"])),
                             bench_seed=spec["seed"] % 97)
        tag = f"chunk {chunk} case {i}: {spec}"
        try:
            cu = run_cuda(case, cfg)
            orc, orc_case = run_oracle(case, cfg)
            assert_decisions_equal(cu, orc, spec["batch"])
            assert_outputs_close(cu, orc, orc_case)
        except AssertionError as exc:
            raise AssertionError(f"{tag}\n{exc}") from exc
        assert ops.query_status() == 0, tag
