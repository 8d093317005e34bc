"""GPU checks of the sink-exclusive prefill ring build (``SINK_EXCLUDE``).

The reference has no implementation of this mode (its hook writes -inf LSEs
under a front sink, ``flashinfer_hooks.py:2205-2215``), so the checks are
  * the CUDA operator against the CPU restatement on the same inputs,
  * the ring rows against attention evaluated directly over ``[min(F,E), E)`` --
    the invariant the reference states for ring rows -- and
  * a decode step that reuses a prefill-written row and must reproduce full
    attention.
"""
import math

import pytest
import torch

from mac_attention_b200 import load_mac_prefill_update_cache_extension, ops
from mac_attention_b200.synth import DecodeCase
from oracle import mac_oracle as O

from helpers import assert_decisions_equal, assert_outputs_close, run_cuda, run_oracle
from prefill_cases import SPECS, make_prompts as _prompts, run_build as _build

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["mma", "tcgen05"])
def sink_kernel(request, monkeypatch):
    """Every test of this file runs on both implementations of the sink-exclusive build: the
    mma.sync kernel (default) and the tcgen05 / tensor-memory kernel."""
    monkeypatch.setenv("MAC_B200_SINK_KERNEL", request.param)
    return request.param


@pytest.mark.parametrize("spec", SPECS, ids=["gqa4_chunked", "gqa8_wrap", "mha_odd_sink", "gqa16"])
def test_sink_exclusive_build_matches_oracle_and_direct_attention(spec):
    ext = load_mac_prefill_update_cache_extension()
    Hq, S, F, M = spec["Hq"], spec["S"], spec["F"], spec["M"]
    t = _prompts(spec["lens"], spec["L0s"], Hq, spec["Hkv"], S, F, M, seed=5)
    want_o, want_l = t.pop("want_o"), t.pop("want_l")
    cpu = {k: v.clone() for k, v in t.items()}
    _build(O.prefill_build, cpu, M, Hq, S, F)
    gpu = {k: v.cuda() for k, v in t.items()}
    _build(ext.mac_prefill_downdate_update_cache, gpu, M, Hq, S, F)
    torch.cuda.synchronize()
    g = {k: v.cpu() for k, v in gpu.items()}
    # copies and integer state: identical
    for name in ("q_cache", "q_post_cache"):
        assert torch.equal(g[name].view(torch.int16), cpu[name].view(torch.int16)), name
    for name in ("request_length", "ready", "cache_epoch"):
        assert torch.equal(g[name], cpu[name]), name
    # states: same empty rows, close values
    fin = torch.isfinite(cpu["lse_cache"])
    assert torch.equal(torch.isfinite(g["lse_cache"]), fin)
    assert torch.allclose(g["lse_cache"][fin], cpu["lse_cache"][fin], rtol=0, atol=2e-3)
    assert O.rel_l2(g["attn_cache"].float(), cpu["attn_cache"].float()) <= 1e-2
    # the rows in the ring against attention taken directly over [min(F,E), E).
    # A downdate amplifies the bf16 rounding of its inputs by (mass of the whole
    # prefix) / (mass left); rows that keep under a fifth of the mass are only
    # checked for a finite result.
    got_o, got_l, ref_o, ref_l, cond = [], [], [], [], []
    for b, (n, L0) in enumerate(zip(spec["lens"], spec["L0s"])):
        start = max(n - M, 0)
        base = int(t["offsets"][b])
        for i in range(start, n):
            pos = L0 + i
            slot = pos % M
            E = max(pos + 1 - S, 0)
            row_o, row_l = g["attn_cache"][b, slot].float(), g["lse_cache"][b, slot]
            assert torch.equal(g["q_cache"][b, slot], t["src_q"][base + i])
            if E <= F:
                assert torch.isinf(row_l).all() and (row_l < 0).all()
                assert (row_o == 0).all()
                continue
            got_o.append(row_o), got_l.append(row_l)
            ref_o.append(want_o[base + i].float()), ref_l.append(want_l[base + i].float())
            cond.append(want_l[base + i].float() - t["full_lse"][base + i])
    got_o, got_l, ref_o, ref_l = map(torch.stack, (got_o, got_l, ref_o, ref_l))
    well = torch.stack(cond) > math.log(0.2)
    assert well.sum() > 0.3 * well.numel()
    assert torch.isfinite(got_l[well]).all()
    assert (got_l[well] - ref_l[well]).abs().max() <= 1e-2
    err = (got_o[well] - ref_o[well]).norm(dim=-1) / ref_o[well].norm(dim=-1)
    assert err.max() <= 6e-2 and err.mean() <= 1e-2, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("F", [64, 0])
def test_decode_reuses_a_prefill_written_row(F):
    """Prefill through the one-pass build (sink-exclusive rows for F = 64, plain rows for
    F = 0), then one decode step whose pre-RoPE query repeats an earlier prompt position:
    every head hits that row, and the merged output (sink + reused prefix + band + tail)
    is full attention."""
    ext = load_mac_prefill_update_cache_extension()
    Hq, Hkv, S, M, L = 8, 2, 16, 512, 400
    t = _prompts([L], [0], Hq, Hkv, S, F, M, seed=9)
    t.pop("want_o"), t.pop("want_l")
    gpu = {k: v.cuda() for k, v in t.items()}
    if F > 0:
        _build(ext.mac_prefill_downdate_update_cache, gpu, M, Hq, S, F)
    else:
        ext.mac_prefill_downdate_update_cache(
            gpu["q_cache"], gpu["attn_cache"], gpu["lse_cache"], gpu["request_length"],
            gpu["req_ids"], gpu["src_q"], gpu["full_attn"], gpu["full_lse"], gpu["band_attn"],
            gpu["band_lse"], gpu["offsets"], gpu["lens"], M, Hq, 128, gpu["q_post_cache"],
            ready=gpu["ready"], cache_epoch=gpu["cache_epoch"], request_epoch=gpu["request_epoch"])
    torch.cuda.synchronize()
    assert bool(gpu["ready"][0])
    pstar = 300
    g = torch.Generator().manual_seed(1)
    new_k = torch.randn(1, Hkv, 128, generator=g).to(torch.bfloat16)
    new_v = torch.randn(1, Hkv, 128, generator=g).to(torch.bfloat16)
    loc = int(t["req_to_token"][0, L])
    k, v = t["k"].clone(), t["v"].clone()
    k[loc], v[loc] = new_k[0], new_v[0]
    case = DecodeCase(
        q_post=t["q_post"][pstar:pstar + 1].clone(), q_pre=t["src_q"][pstar:pstar + 1].clone(),
        k=k, v=v, req_to_token=t["req_to_token"], req_ids=torch.zeros(1, dtype=torch.int32),
        past_lens=torch.tensor([L], dtype=torch.int32),
        out_cache_loc=torch.tensor([loc], dtype=torch.int64),
        query_cache=gpu["q_cache"].cpu(), attn_cache=gpu["attn_cache"].cpu(),
        lse_cache=gpu["lse_cache"].cpu())
    cfg = O.DecodeConfig(max_context=2048, semantic_pos_ahead=S, front_sink_tokens=F,
                         gen_min_limit=0)
    cu = run_cuda(case, cfg)
    orc, orc_case = run_oracle(case, cfg)
    assert_decisions_equal(cu, orc, 1)
    assert_outputs_close(cu, orc, orc_case)
    assert int(cu.ws[3][0].sum()) == Hq                       # every head hit ...
    assert (cu.ws[5][0].cpu() == pstar).all()                 # ... the repeated position
    # full attention over [0, L] with the same post-RoPE query
    G = Hq // Hkv
    tok = t["req_to_token"][0, :L + 1].long()
    kk = k[tok].double().repeat_interleave(G, dim=1).permute(1, 0, 2)
    vv = v[tok].double().repeat_interleave(G, dim=1).permute(1, 0, 2)
    sc = torch.einsum("hd,htd->ht", case.q_post[0].double(), kk) / math.sqrt(128)
    want = torch.einsum("ht,htd->hd", torch.softmax(sc, dim=-1), vv)
    assert O.rel_l2(cu.out[0].float().cpu(), want.float()) <= 3e-2


def test_sink_exclusive_argument_errors():
    ext = load_mac_prefill_update_cache_extension()
    t = _prompts([20], [0], 8, 2, 4, 16, 32, seed=2)
    t.pop("want_o"), t.pop("want_l")
    gpu = {k: v.cuda() for k, v in t.items()}
    with pytest.raises(RuntimeError, match="front_sink_tokens"):
        _build(ext.mac_prefill_downdate_update_cache, gpu, 32, 8, 4, 200)
    bad = dict(gpu)
    bad["q_post"] = None
    with pytest.raises(RuntimeError, match="q_post is required"):
        _build(ext.mac_prefill_downdate_update_cache, bad, 32, 8, 4, 16)
    bad = dict(gpu)
    bad["k"] = gpu["k"][:, :1].contiguous().expand(-1, 3, -1).contiguous()   # Hkv = 3: 8 % 3 != 0
    bad["v"] = bad["k"]
    with pytest.raises(RuntimeError, match="divisible"):
        _build(ext.mac_prefill_downdate_update_cache, bad, 32, 8, 4, 16)


def test_request_without_a_page_table_row_is_reported_and_left_unbuilt():
    """A request id that is a valid ring row but has no row in ``req_to_token`` cannot get
    its sink attention: its ring rows stay as they were, it is NOT marked ready, its length
    is not bumped, and the sticky status word reports a bad request.  The other request of
    the batch is built as usual.  (The access is guarded; nothing faults.)"""
    ext = load_mac_prefill_update_cache_extension()
    Hq, Hkv, S, F, M = 8, 2, 8, 32, 64
    t = _prompts([70, 50], [0, 0], Hq, Hkv, S, F, M, seed=9)
    t.pop("want_o"), t.pop("want_l")
    # three ring rows, two page-table rows; the second prompt claims ring row 2
    for name in ("q_cache", "attn_cache", "lse_cache", "q_post_cache"):
        t[name] = torch.cat([t[name], t[name][:1].clone()])
    t["ready"] = torch.zeros(3, dtype=torch.bool)
    t["cache_epoch"] = torch.full((3,), -1, dtype=torch.int64)
    t["request_epoch"] = torch.arange(3, dtype=torch.int64) + 2
    t["request_length"] = torch.zeros(3, dtype=torch.int32)
    t["req_ids"] = torch.tensor([0, 2], dtype=torch.int32)
    gpu = {k: v.cuda() for k, v in t.items()}
    assert ops.query_status() == 0
    _build(ext.mac_prefill_downdate_update_cache, gpu, M, Hq, S, F)
    torch.cuda.synchronize()
    status = ops.query_status()
    assert status & 0x2, status                       # MAC_B200_STATUS_BAD_REQUEST
    assert ops.query_status() == 0                    # read clears it
    assert gpu["ready"].cpu().tolist() == [True, False, False]
    assert gpu["request_length"].cpu().tolist() == [70, 0, 0]
    assert torch.equal(gpu["q_cache"][2].cpu(), t["q_cache"][2])
    assert torch.equal(gpu["attn_cache"][2].cpu(), t["attn_cache"][2])
    assert not torch.equal(gpu["q_cache"][0].cpu(), t["q_cache"][0])     # request 0 was built


def test_one_pass_build_replays_from_a_cuda_graph():
    ext = load_mac_prefill_update_cache_extension()
    spec = SPECS[0]
    Hq, S, F, M = spec["Hq"], spec["S"], spec["F"], spec["M"]
    t = _prompts(spec["lens"], spec["L0s"], Hq, spec["Hkv"], S, F, M, seed=6)
    t.pop("want_o"), t.pop("want_l")
    # by-batch lengths: the build leaves request_length alone, so a replay repeats the same write
    eager = {k: v.cuda() for k, v in t.items()}
    _build(ext.mac_prefill_downdate_update_cache, eager, M, Hq, S, F)
    torch.cuda.synchronize()
    g = {k: v.cuda() for k, v in t.items()}
    lengths = g["request_length"].clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g["request_length"].copy_(lengths)
        _build(ext.mac_prefill_downdate_update_cache, g, M, Hq, S, F)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for name in ("q_cache", "attn_cache", "q_post_cache"):     # bit patterns: the stamp is NaN
        assert torch.equal(g[name].view(torch.int16), eager[name].view(torch.int16)), name
    assert torch.equal(g["request_length"], eager["request_length"])
    assert torch.equal(g["lse_cache"].view(torch.int32), eager["lse_cache"].view(torch.int32))
    assert ops.query_status() == 0


@pytest.mark.parametrize("chunk", range(3))
def test_sink_exclusive_random_matrix(chunk):
    """Seeded random prompts (GQA group, sink size, window, ring size, chunked prefill
    offsets) through the sink-exclusive build against the CPU restatement."""
    import random

    ext = load_mac_prefill_update_cache_extension()
    rng = random.Random(700 + chunk)
    for i in range(8):
        hkv = rng.choice([1, 2, 4])
        G = rng.choice([1, 2, 4, 8, 16])
        S = rng.choice([1, 4, 16, 64])
        F = rng.choice([0, 1, 16, 20, 64, 128])
        M = rng.choice([16, 64, 128, 300])
        B = rng.randint(1, 3)
        lens = [rng.randint(1, 260) for _ in range(B)]
        L0s = [rng.choice([0, rng.randint(0, 200)]) for _ in range(B)]
        tag = f"chunk {chunk} case {i}: hkv{hkv} G{G} S{S} F{F} M{M} lens{lens} L0{L0s}"
        t = _prompts(lens, L0s, hkv * G, hkv, S, F, M, seed=50 * chunk + i)
        t.pop("want_o"), t.pop("want_l")
        cpu = {k: v.clone() for k, v in t.items()}
        _build(O.prefill_build, cpu, M, hkv * G, S, F)
        gpu = {k: v.cuda() for k, v in t.items()}
        _build(ext.mac_prefill_downdate_update_cache, gpu, M, hkv * G, S, F)
        torch.cuda.synchronize()
        g = {k: v.cpu() for k, v in gpu.items()}
        assert torch.equal(g["q_cache"].view(torch.int16), cpu["q_cache"].view(torch.int16)), tag
        assert torch.equal(g["q_post_cache"].view(torch.int16), cpu["q_post_cache"].view(torch.int16)), tag
        for name in ("request_length", "ready", "cache_epoch"):
            assert torch.equal(g[name], cpu[name]), (name, tag)
        fin = torch.isfinite(cpu["lse_cache"])
        assert torch.equal(torch.isfinite(g["lse_cache"]), fin), tag
        assert O.rel_l2(g["attn_cache"].float(), cpu["attn_cache"].float()) <= 2e-2, tag
    assert ops.query_status() == 0
