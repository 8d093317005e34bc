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
