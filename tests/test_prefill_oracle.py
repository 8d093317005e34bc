"""CPU checks of the prefill-side oracle: the one-pass ring build restates the
reference hook's operator sequence exactly, and its sink-exclusive mode agrees
with attention evaluated directly over ``[min(F, E), E)`` in float64 (an
independent computation: the oracle subtracts, this one masks)."""
import math

import pytest
import torch

from oracle import mac_oracle as O
from prefill_cases import SPECS, make_prompts, run_build


def _sequence_inputs(seed):
    g = torch.Generator().manual_seed(seed)
    R, M, H, D = 6, 16, 8, 128
    lens, req_ids, L0 = [5, 40, 0, 16], [3, 0, 1, 5], [7, 0, 0, 30, 0, 2]
    rows = sum(lens)
    offsets = torch.zeros(len(lens) + 1, dtype=torch.int32)
    offsets[1:] = torch.tensor(lens).cumsum(0)
    full_lse = torch.randn(rows, H, generator=g) + 3
    band_lse = full_lse - torch.rand(rows, H, generator=g) * 4 - 0.05
    band_lse[0, 0] = full_lse[0, 0]
    band_lse[1, 0] = full_lse[1, 0] + 1
    band_lse[2, 0] = float("-inf")
    return dict(
        q_cache=torch.randn(R, M, H, D, generator=g).to(torch.bfloat16),
        attn_cache=torch.randn(R, M, H, D, generator=g).to(torch.bfloat16),
        lse_cache=torch.randn(R, M, H, generator=g),
        q_post_cache=torch.zeros(R, M, H, D, dtype=torch.bfloat16),
        request_length=torch.tensor(L0, dtype=torch.int32),
        req_ids=torch.tensor(req_ids, dtype=torch.int32), offsets=offsets,
        lens=torch.tensor(lens, dtype=torch.int32),
        src_q=torch.randn(rows, H, D, generator=g).to(torch.bfloat16),
        full_attn=torch.randn(rows, H, D, generator=g).to(torch.bfloat16),
        band_attn=torch.randn(rows, H, D, generator=g).to(torch.bfloat16),
        full_lse=full_lse, band_lse=band_lse,
        ready=torch.zeros(R, dtype=torch.bool), cache_epoch=torch.full((R,), -1, dtype=torch.int64),
        request_epoch=torch.arange(R, dtype=torch.int64) + 5), M, H, D


@pytest.mark.parametrize("unmatchable", [False, True])
def test_one_pass_build_equals_the_operator_sequence(unmatchable):
    t, M, H, D = _sequence_inputs(3)
    a = {k: v.clone() for k, v in t.items()}
    lse2 = a["band_lse"] * 0.7
    O.update_then_downdate(a["full_attn"], a["full_lse"], a["band_attn"], lse2)
    if unmatchable:
        lse2 = torch.full_like(lse2, float("-inf"))
    O.prefill_update_cache(a["q_cache"], a["attn_cache"], a["lse_cache"], a["request_length"],
                           a["req_ids"], a["src_q"], a["band_attn"], lse2, a["offsets"], a["lens"],
                           M, H, D, a["q_post_cache"])
    O.mark_persistent_ready(a["ready"], a["cache_epoch"], a["request_epoch"], a["req_ids"])
    b = {k: v.clone() for k, v in t.items()}
    O.prefill_build(b["q_cache"], b["attn_cache"], b["lse_cache"], b["request_length"],
                    b["req_ids"], b["src_q"], b["full_attn"], b["full_lse"], b["band_attn"],
                    b["band_lse"], b["offsets"], b["lens"], M, H, D, b["q_post_cache"],
                    band_lse_scale=0.7, sink_mode=1 if unmatchable else 0, ready=b["ready"],
                    cache_epoch=b["cache_epoch"], request_epoch=b["request_epoch"])
    for k in ("q_cache", "attn_cache", "q_post_cache"):
        assert torch.equal(a[k].view(torch.int16), b[k].view(torch.int16)), k
    for k in ("request_length", "ready", "cache_epoch"):
        assert torch.equal(a[k], b[k]), k
    assert torch.equal(a["lse_cache"].view(torch.int32), b["lse_cache"].view(torch.int32))
    assert torch.equal(b["band_attn"], t["band_attn"])      # inputs untouched


@pytest.mark.parametrize("spec", SPECS, ids=["gqa4_chunked", "gqa8_wrap", "mha_odd_sink", "gqa16"])
def test_sink_exclusive_rows_cover_exactly_the_non_sink_prefix(spec):
    Hq, S, F, M = spec["Hq"], spec["S"], spec["F"], spec["M"]
    t = make_prompts(spec["lens"], spec["L0s"], Hq, spec["Hkv"], S, F, M, seed=5)
    want_o, want_l = t.pop("want_o"), t.pop("want_l")
    run_build(O.prefill_build, t, M, Hq, S, F)
    errs, lerr, empty = [], [], 0
    for b, (n, L0) in enumerate(zip(spec["lens"], spec["L0s"])):
        base = int(t["offsets"][b])
        for i in range(max(n - M, 0), n):
            pos = L0 + i
            E = max(pos + 1 - S, 0)
            ro, rl = t["attn_cache"][b, pos % M].float(), t["lse_cache"][b, pos % M]
            if E <= F:
                assert torch.isinf(rl).all() and (rl < 0).all() and (ro == 0).all()
                empty += 1
                continue
            wo, wl = want_o[base + i].float(), want_l[base + i].float()
            well = (wl - t["full_lse"][base + i]) > math.log(0.2)   # downdate conditioning
            errs.append(((ro - wo).norm(dim=-1) / wo.norm(dim=-1))[well])
            lerr.append((rl - wl).abs()[well])
    e, l = torch.cat(errs), torch.cat(lerr)
    assert e.numel() > 100
    assert float(e.max()) <= 6e-2 and float(e.mean()) <= 1e-2
    assert float(l.max()) <= 1e-3
    assert bool(t["ready"].all())
