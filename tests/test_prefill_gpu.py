"""GPU parity of the prefill-side ring build and the readiness-gate kernels:
bit-exact against the CPU oracle (pure copies and integer updates)."""
import pytest
import torch

from mac_attention_b200 import load_mac_prefill_update_cache_extension
from oracle import mac_oracle as O

pytestmark = pytest.mark.gpu


def _prefill_inputs(R, M, H, D, lens, req_ids, L0, seed, with_post=True, by_batch=False):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    rows = sum(max(x, 0) for x in lens)
    offsets = torch.zeros(B + 1, dtype=torch.int32)
    for b in range(B):
        offsets[b + 1] = offsets[b] + max(lens[b], 0)
    t = dict(
        q_cache=torch.randn(R, M, H, D, generator=g).to(torch.bfloat16),
        attn_cache=torch.randn(R, M, H, D, generator=g).to(torch.bfloat16),
        lse_cache=torch.randn(R, M, H, generator=g),
        request_length=(torch.tensor(L0, dtype=torch.int32)),
        req_ids=torch.tensor(req_ids, dtype=torch.int32),
        src_q=torch.randn(rows, H, D, generator=g).to(torch.bfloat16),
        src_attn=torch.randn(rows, H, D, generator=g).to(torch.bfloat16),
        src_lse=torch.randn(rows, H, generator=g),
        offsets=offsets, lens=torch.tensor(lens, dtype=torch.int32),
    )
    t["q_post_cache"] = torch.zeros(R, M, H, D, dtype=torch.bfloat16) if with_post else torch.empty(0, dtype=torch.bfloat16)
    return t


@pytest.mark.parametrize("spec", [
    dict(R=6, M=16, H=8, D=128, lens=[5, 40, 0, 16], req_ids=[3, 0, 1, 5], L0=[7, 0, 0, 30, 0, 2]),
    dict(R=4, M=512, H=32, D=128, lens=[2048, 100, 513], req_ids=[2, 9, 0], L0=[0, 0, 100, 0]),
    dict(R=3, M=8, H=3, D=16, lens=[9, 3], req_ids=[1, -1], L0=[0, -5, 0]),
    dict(R=5, M=32, H=4, D=128, lens=[10, 50, 7], req_ids=[4, 2, 0], L0=[3, 64, 9], by_batch=True),
], ids=["small", "qwen_ring", "odd_rows_bad_req", "length_by_batch"])
def test_prefill_update_cache_bit_exact(spec):
    ext = load_mac_prefill_update_cache_extension()
    by_batch = spec.get("by_batch", False)
    t = _prefill_inputs(spec["R"], spec["M"], spec["H"], spec["D"], spec["lens"], spec["req_ids"],
                        spec["L0"], seed=1, by_batch=by_batch)
    cpu = {k: v.clone() for k, v in t.items()}
    O.prefill_update_cache(cpu["q_cache"], cpu["attn_cache"], cpu["lse_cache"],
                           cpu["request_length"], cpu["req_ids"], cpu["src_q"], cpu["src_attn"],
                           cpu["src_lse"], cpu["offsets"], cpu["lens"], spec["M"], spec["H"],
                           spec["D"], cpu["q_post_cache"])
    gpu = {k: v.cuda() for k, v in t.items()}
    ext.mac_prefill_update_cache(gpu["q_cache"], gpu["attn_cache"], gpu["lse_cache"],
                                 gpu["request_length"], gpu["req_ids"], gpu["src_q"],
                                 gpu["src_attn"], gpu["src_lse"], gpu["offsets"], gpu["lens"],
                                 spec["M"], spec["H"], spec["D"], gpu["q_post_cache"])
    torch.cuda.synchronize()
    for name in ("q_cache", "attn_cache", "q_post_cache", "request_length"):
        a, b = gpu[name].cpu(), cpu[name]
        if a.dtype == torch.bfloat16:
            a, b = a.view(torch.int16), b.view(torch.int16)
        assert torch.equal(a, b), name
    assert torch.equal(gpu["lse_cache"].cpu().view(torch.int32), cpu["lse_cache"].view(torch.int32))


def test_prefill_noop_and_errors():
    ext = load_mac_prefill_update_cache_extension()
    t = {k: v.cuda() for k, v in _prefill_inputs(2, 4, 2, 128, [3], [0], [0, 0], 0).items()}
    before = t["q_cache"].clone()
    ext.mac_prefill_update_cache(t["q_cache"], t["attn_cache"], t["lse_cache"], t["request_length"],
                                 t["req_ids"], t["src_q"], t["src_attn"], t["src_lse"],
                                 t["offsets"], t["lens"], 0, 2, 128, t["q_post_cache"])
    torch.cuda.synchronize()
    assert torch.equal(before, t["q_cache"])
    with pytest.raises(RuntimeError, match="capacity"):
        ext.mac_prefill_update_cache(t["q_cache"], t["attn_cache"], t["lse_cache"],
                                     t["request_length"], t["req_ids"], t["src_q"], t["src_attn"],
                                     t["src_lse"], t["offsets"], t["lens"], 8, 2, 128,
                                     t["q_post_cache"])
    with pytest.raises(RuntimeError, match="wrong dtype"):
        ext.mac_prefill_update_cache(t["q_cache"].float(), t["attn_cache"], t["lse_cache"],
                                     t["request_length"], t["req_ids"], t["src_q"], t["src_attn"],
                                     t["src_lse"], t["offsets"], t["lens"], 4, 2, 128,
                                     t["q_post_cache"])


def test_gate_and_request_state_kernels_bit_exact():
    ext = load_mac_prefill_update_cache_extension()
    R = 300
    g = torch.Generator().manual_seed(3)
    ready = torch.rand(R, generator=g) < 0.5
    ce = torch.randint(-1, 4, (R,), generator=g, dtype=torch.int64)
    re_ = torch.randint(0, 4, (R,), generator=g, dtype=torch.int64)
    ids = (torch.randperm(R + 5, generator=g) - 2).to(torch.int32)  # unique, some out of range
    c = [x.clone() for x in (ready, ce, re_)]
    d = [x.cuda() for x in (ready, ce, re_)]
    O.mark_persistent_ready(c[0], c[1], c[2], ids[:60])
    ext.mac_mark_persistent_ready(d[0], d[1], d[2], ids[:60].cuda())
    O.invalidate_persistent_ready(c[0], c[1], c[2], ids[40:120])
    ext.mac_invalidate_persistent_ready(d[0], d[1], d[2], ids[40:120].cuda())
    torch.cuda.synchronize()
    for x, y in zip(c, d):
        assert torch.equal(x, y.cpu())
    B = 150
    req_len = torch.zeros(R, dtype=torch.int32)
    mreq = torch.zeros(R, dtype=torch.int32)
    cl = torch.zeros(B, dtype=torch.int32)
    seq = torch.randint(0, 5000, (B,), generator=g, dtype=torch.int32)
    cur = torch.randint(0, 5000, (B,), generator=g, dtype=torch.int32)
    rid = ids[:B].contiguous()
    cc = [req_len.clone(), mreq.clone(), cl.clone()]
    dd = [req_len.cuda(), mreq.cuda(), cl.cuda()]
    O.update_request_state(cc[0], cc[1], cc[2], rid, seq, cur)
    ext.mac_update_request_state(dd[0], dd[1], dd[2], rid.cuda(), seq.cuda(), cur.cuda())
    torch.cuda.synchronize()
    for x, y in zip(cc, dd):
        assert torch.equal(x, y.cpu())


def test_prefill_then_decode_hits_the_prefill_rows():
    """Ring built by the prefill operator is what the decode step matches against."""
    from mac_attention_b200 import synth
    from tests.helpers import assert_decisions_equal, assert_outputs_close, run_cuda, run_oracle

    ext = load_mac_prefill_update_cache_extension()
    case = synth.make_decode_case(batch=2, ctx=1000, hq=16, hkv=4, capacity=128, seed=6)
    H, D, M = 16, 128, 128
    lens = [1000, 1000]
    g = torch.Generator().manual_seed(8)
    src_q = torch.randn(2000, H, D, generator=g).to(torch.bfloat16)
    # last prompt row of request 0 is a near-duplicate of its step query
    src_q[999] = (case.q_pre[0].float() + 0.05 * torch.randn(H, D, generator=g)).to(torch.bfloat16)
    src_attn = torch.randn(2000, H, D, generator=g).to(torch.bfloat16)
    src_lse = torch.randn(2000, H, generator=g) + 4
    rl = torch.zeros(2, dtype=torch.int32)
    offsets = torch.tensor([0, 1000, 2000], dtype=torch.int32)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    cpu = case.clone()
    O.prefill_update_cache(cpu.query_cache, cpu.attn_cache, cpu.lse_cache, rl.clone(), cpu.req_ids,
                           src_q, src_attn, src_lse, offsets, lens_t, M, H, D, None)
    gpu = case.to("cuda")
    ext.mac_prefill_update_cache(gpu.query_cache, gpu.attn_cache, gpu.lse_cache, rl.cuda(),
                                 gpu.req_ids, src_q.cuda(), src_attn.cuda(), src_lse.cuda(),
                                 offsets.cuda(), lens_t.cuda(), M, H, D,
                                 torch.empty(0, device="cuda", dtype=torch.bfloat16))
    torch.cuda.synchronize()
    assert torch.equal(gpu.query_cache.cpu().view(torch.int16), cpu.query_cache.view(torch.int16))
    cfg = O.DecodeConfig(max_context=2048, semantic_pos_ahead=64)
    cu = run_cuda(gpu, cfg)
    orc, orc_case = run_oracle(cpu, cfg)
    assert_decisions_equal(cu, orc, 2)
    assert cu.ws[3][0].sum() == H and (cu.ws[5][0] == 999).all() and cu.ws[3][1].sum() == 0
    assert_outputs_close(cu, orc, orc_case)


# --------------------------------------------------------------------------
# One-pass build: downdate + ring write + ready mark
# --------------------------------------------------------------------------
def _build_inputs(R, M, H, D, lens, req_ids, L0, seed, lse_dtypes=(torch.float32, torch.float32)):
    t = _prefill_inputs(R, M, H, D, lens, req_ids, L0, seed)
    g = torch.Generator().manual_seed(seed + 100)
    rows = t["src_q"].shape[0]
    t["full_attn"] = t.pop("src_attn")
    full_lse = torch.randn(rows, H, generator=g) + 3.0
    band_lse = full_lse - torch.rand(rows, H, generator=g) * 4.0 - 0.05
    if rows >= 4:
        band_lse[0, 0] = full_lse[0, 0]            # band is the whole prefix -> empty state
        band_lse[1, 0] = full_lse[1, 0] + 1.0      # inconsistent pair -> keep the full state
        band_lse[2, 0] = float("-inf")             # empty band
        band_lse[rows - 1, H - 1] = full_lse[rows - 1, H - 1]
    t.pop("src_lse")
    t["full_lse"] = full_lse.to(lse_dtypes[0])
    t["band_lse"] = band_lse.to(lse_dtypes[1])
    t["band_attn"] = torch.randn(rows, H, D, generator=g).to(torch.bfloat16)
    t["ready"] = torch.zeros(R, dtype=torch.bool)
    t["cache_epoch"] = torch.full((R,), -1, dtype=torch.int64)
    t["request_epoch"] = torch.arange(R, dtype=torch.int64) + 5
    return t


def _sequential(mod, t, M, H, D, scale, unmatchable):
    """The reference hook's sequence of operators, on the tensors of ``t`` (modified)."""
    band_lse = (t["band_lse"].float() * scale).to(t["band_lse"].dtype) if scale != 1.0 else t["band_lse"]
    mod["downdate"](t["full_attn"], t["full_lse"], t["band_attn"], band_lse)
    lse32 = band_lse.float()
    if unmatchable:
        lse32 = torch.full_like(lse32, float("-inf"))
    mod["prefill"](t["q_cache"], t["attn_cache"], t["lse_cache"], t["request_length"],
                   t["req_ids"], t["src_q"], t["band_attn"], lse32.contiguous(), t["offsets"], t["lens"],
                   M, H, D, t["q_post_cache"])
    mod["mark"](t["ready"], t["cache_epoch"], t["request_epoch"], t["req_ids"])


@pytest.mark.parametrize("spec", [
    dict(R=6, M=16, H=8, D=128, lens=[5, 40, 0, 16], req_ids=[3, 0, 1, 5], L0=[7, 0, 0, 30, 0, 2]),
    dict(R=4, M=512, H=32, D=128, lens=[2048, 100, 513], req_ids=[2, 9, 0], L0=[0, 0, 100, 0]),
    dict(R=3, M=8, H=3, D=20, lens=[9, 3], req_ids=[1, -1], L0=[0, -5, 0]),
    dict(R=3, M=64, H=40, D=64, lens=[70, 33], req_ids=[2, 0], L0=[11, 0, 50], scale=0.6931471805599453),
    dict(R=5, M=32, H=4, D=128, lens=[10, 50, 7], req_ids=[4, 2, 0], L0=[3, 64, 9], unmatchable=True),
    dict(R=2, M=32, H=8, D=128, lens=[40, 20], req_ids=[1, 0], L0=[0, 0],
         lse_dtypes=(torch.bfloat16, torch.float16)),
], ids=["small", "qwen_ring", "odd_dims_bad_req", "ln2_scale", "unmatchable", "narrow_lse"])
def test_prefill_build_matches_the_operator_sequence(spec):
    ext = load_mac_prefill_update_cache_extension()
    from mac_attention_b200 import ops
    M, H, D = spec["M"], spec["H"], spec["D"]
    scale, unm = spec.get("scale", 1.0), spec.get("unmatchable", False)
    t = _build_inputs(spec["R"], M, H, D, spec["lens"], spec["req_ids"], spec["L0"], seed=3,
                      lse_dtypes=spec.get("lse_dtypes", (torch.float32, torch.float32)))
    # (a) CPU oracle of the sequence (oracle LSE arithmetic is fp32)
    cpu = {k: v.clone() for k, v in t.items()}
    cpu["full_lse"], cpu["band_lse"] = cpu["full_lse"].float(), cpu["band_lse"].float()
    _sequential(dict(downdate=O.update_then_downdate, prefill=O.prefill_update_cache,
                     mark=O.mark_persistent_ready), cpu, M, H, D, scale, unm)
    # (b) the same sequence through the separate CUDA operators
    seq = {k: v.cuda() for k, v in t.items()}
    _sequential(dict(downdate=ops.mac_update_then_downdate_bf16_inplace,
                     prefill=ext.mac_prefill_update_cache, mark=ext.mac_mark_persistent_ready),
                seq, M, H, D, scale, unm)
    # (c) the one-pass operator
    one = {k: v.cuda() for k, v in t.items()}
    band_before = one["band_attn"].clone()
    ext.mac_prefill_downdate_update_cache(
        one["q_cache"], one["attn_cache"], one["lse_cache"], one["request_length"], one["req_ids"],
        one["src_q"], one["full_attn"], one["full_lse"], one["band_attn"], one["band_lse"],
        one["offsets"], one["lens"], M, H, D, one["q_post_cache"], band_lse_scale=scale,
        sink_mode=ops.SINK_UNMATCHABLE if unm else ops.SINK_NONE, ready=one["ready"],
        cache_epoch=one["cache_epoch"], request_epoch=one["request_epoch"])
    torch.cuda.synchronize()
    assert torch.equal(one["band_attn"], band_before)
    narrow = "lse_dtypes" in spec
    for name in ("q_cache", "q_post_cache", "request_length", "ready", "cache_epoch"):
        a, b, c = one[name].cpu(), seq[name].cpu(), cpu[name]
        if a.dtype == torch.bfloat16:
            a, b, c = a.view(torch.int16), b.view(torch.int16), c.view(torch.int16)
        assert torch.equal(a, b), name
        assert torch.equal(a, c), name
    if not narrow:
        # same arithmetic as the separate operators: identical bits
        assert torch.equal(one["attn_cache"].view(torch.int16), seq["attn_cache"].view(torch.int16))
        assert torch.equal(one["lse_cache"].view(torch.int32), seq["lse_cache"].view(torch.int32))
    else:
        # the separate operators round the downdated LSE to its narrow type on the way
        assert O.rel_l2(one["attn_cache"].float().cpu(), seq["attn_cache"].float().cpu()) <= 2e-3
    fin_gpu, fin_cpu = torch.isfinite(one["lse_cache"].cpu()), torch.isfinite(cpu["lse_cache"])
    assert torch.equal(fin_gpu, fin_cpu)
    both = fin_gpu & fin_cpu
    assert torch.allclose(one["lse_cache"].cpu()[both], cpu["lse_cache"][both], rtol=1e-4, atol=2e-2 if narrow else 1e-4)
    assert O.rel_l2(one["attn_cache"].float().cpu(), cpu["attn_cache"].float()) <= 2e-3


def test_prefill_build_argument_errors():
    ext = load_mac_prefill_update_cache_extension()
    t = {k: v.cuda() for k, v in _build_inputs(2, 4, 2, 128, [3], [0], [0, 0], 0).items()}

    def call(**kw):
        a = dict(t)
        a.update(kw)
        extra = {k: a[k] for k in ("ready", "cache_epoch", "request_epoch") if a.get(k) is not None}
        ext.mac_prefill_downdate_update_cache(
            a["q_cache"], a["attn_cache"], a["lse_cache"], a["request_length"], a["req_ids"],
            a["src_q"], a["full_attn"], a["full_lse"], a["band_attn"], a["band_lse"], a["offsets"],
            a["lens"], 4, 2, 128, a["q_post_cache"], sink_mode=a.get("sink_mode", 0), **extra)

    with pytest.raises(RuntimeError, match="band_attn must match"):
        call(band_attn=t["band_attn"][:2].contiguous())
    with pytest.raises(RuntimeError, match="float32, bfloat16, or float16"):
        call(band_lse=t["band_lse"].double())
    with pytest.raises(RuntimeError, match="go together"):
        call(cache_epoch=None)
    with pytest.raises(RuntimeError, match="sink_mode"):
        call(sink_mode=7)
    call()
    torch.cuda.synchronize()
    assert bool(t["ready"][0]) and not bool(t["ready"][1])


def test_prefill_build_matches_the_reference_kernels_in_the_hook_order():
    """Ring contents against the reference's own CUDA operators (built for sm_100a
    from the reference sources), called in the order its prefill hook calls them."""
    from oracle import build_ref

    rdd, rpre = build_ref.load_downdate(), build_ref.load_prefill()
    if rdd is None or rpre is None:
        pytest.skip("reference kernels are not built on this box")
    ext = load_mac_prefill_update_cache_extension()
    R, M, H, D = 4, 512, 32, 128
    lens, req_ids, L0 = [2048, 100, 513], [2, 3, 0], [0, 0, 100, 7]
    t = _build_inputs(R, M, H, D, lens, req_ids, L0, seed=11)
    ln2 = 0.6931471805599453
    ref = {k: v.cuda() for k, v in t.items()}
    band_lse = ref["band_lse"] * ln2
    rdd.mac_update_then_downdate_bf16_inplace(ref["full_attn"], ref["full_lse"], ref["band_attn"],
                                              band_lse)
    rpre.mac_prefill_update_cache(ref["q_cache"], ref["attn_cache"], ref["lse_cache"],
                                  ref["request_length"], ref["req_ids"], ref["src_q"],
                                  ref["band_attn"], band_lse, ref["offsets"], ref["lens"], M, H, D,
                                  ref["q_post_cache"])
    rpre.mac_mark_persistent_ready(ref["ready"], ref["cache_epoch"], ref["request_epoch"],
                                   ref["req_ids"])
    one = {k: v.cuda() for k, v in t.items()}
    ext.mac_prefill_downdate_update_cache(
        one["q_cache"], one["attn_cache"], one["lse_cache"], one["request_length"], one["req_ids"],
        one["src_q"], one["full_attn"], one["full_lse"], one["band_attn"], one["band_lse"],
        one["offsets"], one["lens"], M, H, D, one["q_post_cache"], band_lse_scale=ln2,
        ready=one["ready"], cache_epoch=one["cache_epoch"], request_epoch=one["request_epoch"])
    torch.cuda.synchronize()
    for name in ("q_cache", "q_post_cache"):
        assert torch.equal(one[name].view(torch.int16), ref[name].view(torch.int16)), name
    for name in ("request_length", "ready", "cache_epoch"):
        assert torch.equal(one[name], ref[name]), name
    fin = torch.isfinite(ref["lse_cache"])
    assert torch.equal(torch.isfinite(one["lse_cache"]), fin)
    assert (one["lse_cache"][fin] - ref["lse_cache"][fin]).abs().max() <= 1e-3   # reference: fast-math exp/log
    assert O.rel_l2(one["attn_cache"].float().cpu(), ref["attn_cache"].float().cpu()) <= 1e-2


def test_prefill_build_noop_cases_leave_the_ring_alone():
    ext = load_mac_prefill_update_cache_extension()
    t = {k: v.cuda() for k, v in _build_inputs(2, 4, 2, 128, [3], [0], [0, 0], 0).items()}
    before = {k: t[k].clone() for k in ("q_cache", "attn_cache", "lse_cache", "ready")}

    def call(capacity, **kw):
        a = dict(t)
        a.update(kw)
        ext.mac_prefill_downdate_update_cache(
            a["q_cache"], a["attn_cache"], a["lse_cache"], a["request_length"], a["req_ids"],
            a["src_q"], a["full_attn"], a["full_lse"], a["band_attn"], a["band_lse"], a["offsets"],
            a["lens"], capacity, 2, 128, a["q_post_cache"], ready=a["ready"],
            cache_epoch=a["cache_epoch"], request_epoch=a["request_epoch"])

    call(0)                                                       # capacity <= 0: the reference's silent no-op
    call(4, req_ids=t["req_ids"][:0], lens=t["lens"][:0], offsets=t["offsets"][:1])   # empty batch
    call(4, lens=torch.zeros_like(t["lens"]))                     # zero-length prompt: nothing copied ...
    torch.cuda.synchronize()
    for k in ("q_cache", "attn_cache", "lse_cache"):
        assert torch.equal(before[k].view(torch.uint8), t[k].view(torch.uint8)), k
    assert bool(t["ready"][0])                                    # ... but the request is marked, as by the reference's mark kernel


@pytest.mark.parametrize("chunk", range(4))
def test_prefill_build_random_matrix(chunk):
    """Seeded random geometries of the one-pass build (modes NONE / UNMATCHABLE) against the
    CPU restatement and, bit for bit, against the separate CUDA operators."""
    import random

    from mac_attention_b200 import ops

    ext = load_mac_prefill_update_cache_extension()
    rng = random.Random(300 + chunk)
    for i in range(15):
        R = rng.randint(1, 6)
        M = rng.choice([1, 3, 8, 32, 100, 256])
        H = rng.choice([1, 3, 8, 32, 40])
        D = rng.choice([16, 20, 64, 128])
        B = rng.randint(1, 5)
        lens = [rng.choice([0, 1, rng.randint(1, 40), rng.randint(1, 2 * M + 3)]) for _ in range(B)]
        req_ids = [rng.choice([rng.randint(0, R - 1), rng.randint(0, R - 1), -1, R + 2]) for _ in range(B)]
        # distinct valid request ids (two batch rows writing one ring would race in any implementation)
        seen = set()
        for b in range(B):
            if 0 <= req_ids[b] < R:
                if req_ids[b] in seen:
                    req_ids[b] = -1
                seen.add(req_ids[b])
        L0 = [rng.choice([0, -3, rng.randint(0, 3 * M)]) for _ in range(R)]
        unm = rng.random() < 0.4
        scale = rng.choice([1.0, 0.6931471805599453])
        tag = f"chunk {chunk} case {i}: R{R} M{M} H{H} D{D} lens{lens} req{req_ids} L0{L0} unm{unm}"
        t = _build_inputs(R, M, H, D, lens, req_ids, L0, seed=1000 * chunk + i)
        cpu = {k: v.clone() for k, v in t.items()}
        O.prefill_build(cpu["q_cache"], cpu["attn_cache"], cpu["lse_cache"], cpu["request_length"],
                        cpu["req_ids"], cpu["src_q"], cpu["full_attn"], cpu["full_lse"],
                        cpu["band_attn"], cpu["band_lse"], cpu["offsets"], cpu["lens"], M, H, D,
                        cpu["q_post_cache"], band_lse_scale=scale, sink_mode=1 if unm else 0,
                        ready=cpu["ready"], cache_epoch=cpu["cache_epoch"],
                        request_epoch=cpu["request_epoch"])
        seq = {k: v.cuda() for k, v in t.items()}
        _sequential(dict(downdate=ops.mac_update_then_downdate_bf16_inplace,
                         prefill=ext.mac_prefill_update_cache, mark=ext.mac_mark_persistent_ready),
                    seq, M, H, D, scale, unm)
        one = {k: v.cuda() for k, v in t.items()}
        ext.mac_prefill_downdate_update_cache(
            one["q_cache"], one["attn_cache"], one["lse_cache"], one["request_length"],
            one["req_ids"], one["src_q"], one["full_attn"], one["full_lse"], one["band_attn"],
            one["band_lse"], one["offsets"], one["lens"], M, H, D, one["q_post_cache"],
            band_lse_scale=scale, sink_mode=1 if unm else 0, ready=one["ready"],
            cache_epoch=one["cache_epoch"], request_epoch=one["request_epoch"])
        torch.cuda.synchronize()
        for name in ("q_cache", "attn_cache", "q_post_cache"):
            assert torch.equal(one[name].view(torch.int16), seq[name].view(torch.int16)), (name, tag)
        assert torch.equal(one["lse_cache"].view(torch.int32), seq["lse_cache"].view(torch.int32)), tag
        for name in ("request_length", "ready", "cache_epoch"):
            assert torch.equal(one[name].cpu(), cpu[name]), (name, tag)
            assert torch.equal(one[name], seq[name]), (name, tag)
        assert torch.equal(one["q_cache"].cpu().view(torch.int16), cpu["q_cache"].view(torch.int16)), tag
        fin = torch.isfinite(cpu["lse_cache"])
        assert torch.equal(torch.isfinite(one["lse_cache"]).cpu(), fin), tag
        assert O.rel_l2(one["attn_cache"].float().cpu(), cpu["attn_cache"].float()) <= 2e-3, tag


@pytest.mark.parametrize("chunk", range(3))
def test_prefill_update_cache_random_matrix(chunk):
    """Seeded random geometries of the plain ring copy against the oracle, bit for bit."""
    import random

    ext = load_mac_prefill_update_cache_extension()
    rng = random.Random(20 + chunk)
    for i in range(15):
        R, M = rng.randint(1, 6), rng.choice([1, 3, 8, 32, 100, 256])
        H, D = rng.choice([1, 3, 8, 32, 40]), rng.choice([4, 16, 20, 64, 128])
        B = rng.randint(1, 5)
        lens = [rng.choice([0, 1, rng.randint(1, 40), rng.randint(1, 2 * M + 3)]) for _ in range(B)]
        req_ids, seen = [], set()
        for _ in range(B):
            r = rng.choice([rng.randint(0, R - 1), rng.randint(0, R - 1), -1, R + 2])
            if r in seen:
                r = -1
            seen.add(r)
            req_ids.append(r)
        by_batch = rng.random() < 0.3
        L0 = [rng.choice([0, -3, rng.randint(0, 3 * M)]) for _ in range(B if by_batch else R)]
        if (len(L0) == B) != by_batch:       # R == B makes the operator take the by-batch reading
            continue
        with_post = rng.random() < 0.7
        t = _prefill_inputs(R, M, H, D, lens, req_ids, L0, seed=100 * chunk + i, with_post=with_post)
        cpu = {k: v.clone() for k, v in t.items()}
        O.prefill_update_cache(cpu["q_cache"], cpu["attn_cache"], cpu["lse_cache"],
                               cpu["request_length"], cpu["req_ids"], cpu["src_q"], cpu["src_attn"],
                               cpu["src_lse"], cpu["offsets"], cpu["lens"], M, H, D, cpu["q_post_cache"])
        gpu = {k: v.cuda() for k, v in t.items()}
        ext.mac_prefill_update_cache(gpu["q_cache"], gpu["attn_cache"], gpu["lse_cache"],
                                     gpu["request_length"], gpu["req_ids"], gpu["src_q"],
                                     gpu["src_attn"], gpu["src_lse"], gpu["offsets"], gpu["lens"],
                                     M, H, D, gpu["q_post_cache"])
        torch.cuda.synchronize()
        tag = f"chunk {chunk} case {i}: R{R} M{M} H{H} D{D} lens{lens} req{req_ids} L0{L0}"
        for name in ("q_cache", "attn_cache", "q_post_cache"):
            if gpu[name].numel():
                assert torch.equal(gpu[name].cpu().view(torch.int16), cpu[name].view(torch.int16)), (name, tag)
        assert torch.equal(gpu["request_length"].cpu(), cpu["request_length"]), tag
        assert torch.equal(gpu["lse_cache"].cpu().view(torch.int32), cpu["lse_cache"].view(torch.int32)), tag


def test_prefill_build_at_serving_size_equals_the_operator_sequence():
    """8 prompts of 32768 tokens, Hq 32, D 128, ring 2048 (the serving geometry of the
    benchmark, an eighth of its batch): the one-pass build leaves bit for bit the ring the
    separate downdate + copy + mark operators leave, wrap-around and chunk offsets included."""
    from mac_attention_b200 import ops

    ext = load_mac_prefill_update_cache_extension()
    B, plen, H, D, M = 8, 32768, 32, 128, 2048
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(12)

    def rnd(*shape):
        return torch.randn(*shape, device=dev, generator=g)

    src_q = rnd(B * plen, H, D).to(torch.bfloat16)
    full = rnd(B * plen, H, D).to(torch.bfloat16)
    band = rnd(B * plen, H, D).to(torch.bfloat16)
    full_lse = rnd(B * plen, H) + 8
    band_lse = (full_lse - torch.rand(B * plen, H, device=dev, generator=g) * 4 - 0.1) / 0.6931471805599453
    req_ids = torch.tensor([5, 2, 7, 0, 3, 6, 1, 4], device=dev, dtype=torch.int32)
    offsets = (torch.arange(B + 1, device=dev, dtype=torch.int32) * plen).contiguous()
    lens = torch.full((B,), plen, device=dev, dtype=torch.int32)
    L0 = torch.tensor([0, 777, 4096, 1, 2047, 100000, 31, 8191], device=dev, dtype=torch.int32)

    def fresh():
        return dict(q=torch.zeros(B, M, H, D, device=dev, dtype=torch.bfloat16),
                    a=torch.zeros(B, M, H, D, device=dev, dtype=torch.bfloat16),
                    l=torch.zeros(B, M, H, device=dev), p=torch.zeros(B, M, H, D, device=dev, dtype=torch.bfloat16),
                    rl=L0.clone(), ready=torch.zeros(B, device=dev, dtype=torch.bool),
                    ce=torch.full((B,), -1, device=dev, dtype=torch.int64),
                    re=torch.arange(B, device=dev, dtype=torch.int64))

    one = fresh()
    ext.mac_prefill_downdate_update_cache(one["q"], one["a"], one["l"], one["rl"], req_ids, src_q, full,
                                          full_lse, band, band_lse, offsets, lens, M, H, D, one["p"],
                                          band_lse_scale=0.6931471805599453, ready=one["ready"],
                                          cache_epoch=one["ce"], request_epoch=one["re"])
    seq = fresh()
    scaled = band_lse * 0.6931471805599453
    band_work = band.clone()
    ops.mac_update_then_downdate_bf16_inplace(full, full_lse, band_work, scaled)
    ext.mac_prefill_update_cache(seq["q"], seq["a"], seq["l"], seq["rl"], req_ids, src_q, band_work,
                                 scaled, offsets, lens, M, H, D, seq["p"])
    ext.mac_mark_persistent_ready(seq["ready"], seq["ce"], seq["re"], req_ids)
    torch.cuda.synchronize()
    for k in ("q", "a", "p"):
        assert torch.equal(one[k].view(torch.int16), seq[k].view(torch.int16)), k
    assert torch.equal(one["l"].view(torch.int32), seq["l"].view(torch.int32))
    for k in ("rl", "ready", "ce"):
        assert torch.equal(one[k], seq[k]), k
    # every ring slot was written: the last 2048 rows of each prompt, rotated by its offset
    n = 3
    slot = int((L0[n] + plen - 1) % M)
    assert torch.equal(one["q"][int(req_ids[n]), slot], src_q[(n + 1) * plen - 1])
