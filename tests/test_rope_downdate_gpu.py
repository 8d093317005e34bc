"""GPU parity of the two operators either side of the decode path: the fused
decode-time RoPE + pre-RoPE q preserve + KV-pool write, and the prefill-side
LSE downdate.  Checked against the CPU oracle and, when they were built, the
reference's own kernels compiled for sm_100a."""
import math

import pytest
import torch

from mac_attention_b200 import (load_mac_decode_rope_preserve_extension,
                                load_mac_merge_downdate_cache_extension)
from oracle import mac_oracle as O

pytestmark = pytest.mark.gpu


def _rope_inputs(N, Hq, Hkv, D, rot, max_pos, pool, seed, pos_dtype, loc_dtype, fused_qkv=True):
    g = torch.Generator().manual_seed(seed)
    width = (Hq + 2 * Hkv) * D
    if fused_qkv:  # q, k, v are column slices of one projection output, as in serving
        qkv = torch.randn(N, width, generator=g).to(torch.bfloat16)
        q, k, v = qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]
    else:
        qkv = None
        q = torch.randn(N, Hq * D, generator=g).to(torch.bfloat16)
        k = torch.randn(N, Hkv * D, generator=g).to(torch.bfloat16)
        v = torch.randn(N, Hkv * D, generator=g).to(torch.bfloat16)
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2).float() / rot))
    ang = torch.arange(max_pos).float()[:, None] * inv[None, :]
    cache = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()
    positions = torch.randint(0, max_pos, (N,), generator=g).to(pos_dtype)
    locs = torch.randperm(pool, generator=g)[:N].to(loc_dtype)
    return dict(qkv=qkv, q=q, k=k, v=v, q_pre=torch.zeros(N + 2, Hq, D, dtype=torch.bfloat16),
                k_buffer=torch.zeros(pool, Hkv, D, dtype=torch.bfloat16),
                v_buffer=torch.zeros(pool, Hkv, D, dtype=torch.bfloat16), cache=cache,
                positions=positions, locs=locs)


def _to_cuda(t, Hq, Hkv, D):
    out = {}
    if t["qkv"] is not None:
        qkv = t["qkv"].cuda()
        out["qkv"] = qkv
        out["q"], out["k"], out["v"] = (qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D],
                                        qkv[:, (Hq + Hkv) * D:])
    else:
        out["qkv"] = None
        out["q"], out["k"], out["v"] = t["q"].cuda(), t["k"].cuda(), t["v"].cuda()
    for name in ("q_pre", "k_buffer", "v_buffer", "cache", "positions", "locs"):
        out[name] = t[name].cuda()
    return out


def _run_rope(ext, t, D, neox):
    ext.mac_decode_rope_preserve_q_bf16(t["q"], t["k"], t["v"], t["q_pre"], t["k_buffer"],
                                        t["v_buffer"], t["cache"], t["positions"], t["locs"], D,
                                        neox)


def _ulp_close(a, b, max_frac=2e-3):
    """bf16 results equal except for a few values one bf16 step apart (fused vs
    unfused rounding of the two products)."""
    ai, bi = a.view(torch.int16).int(), b.view(torch.int16).int()
    diff = (ai - bi).abs()
    assert int(diff.max()) <= 1, f"max bf16 step difference {int(diff.max())}"
    assert float((diff > 0).float().mean()) <= max_frac


@pytest.mark.parametrize("spec", [
    dict(N=64, Hq=32, Hkv=8, D=128, rot=128, neox=True, pos=torch.int64, loc=torch.int64),
    dict(N=5, Hq=32, Hkv=4, D=128, rot=128, neox=False, pos=torch.int32, loc=torch.int32),
    dict(N=17, Hq=8, Hkv=2, D=128, rot=64, neox=True, pos=torch.int64, loc=torch.int32),
    dict(N=3, Hq=4, Hkv=4, D=64, rot=32, neox=False, pos=torch.int32, loc=torch.int64),
    dict(N=7, Hq=6, Hkv=2, D=40, rot=20, neox=True, pos=torch.int64, loc=torch.int64, fused=False),
], ids=["llama8b", "qwen_interleaved", "partial_rotary", "d64", "odd_dims_scalar_path"])
def test_rope_preserve_matches_oracle_and_reference(spec):
    ext = load_mac_decode_rope_preserve_extension()
    t = _rope_inputs(spec["N"], spec["Hq"], spec["Hkv"], spec["D"], spec["rot"], 4096, 500, 3,
                     spec["pos"], spec["loc"], fused_qkv=spec.get("fused", True))
    gpu = _to_cuda(t, spec["Hq"], spec["Hkv"], spec["D"])
    q_before = t["q"].clone()
    O.decode_rope_preserve(t["q"], t["k"], t["v"], t["q_pre"], t["k_buffer"], t["v_buffer"],
                           t["cache"], t["positions"], t["locs"], spec["D"], spec["neox"])
    _run_rope(ext, gpu, spec["D"], spec["neox"])
    torch.cuda.synchronize()
    N = spec["N"]
    # copies are exact
    assert torch.equal(gpu["q_pre"].cpu()[:N].view(N, -1).view(torch.int16), q_before.contiguous().view(torch.int16))
    assert torch.equal(gpu["q_pre"].cpu()[N:], torch.zeros_like(t["q_pre"][N:]))
    assert torch.equal(gpu["v_buffer"].cpu().view(torch.int16), t["v_buffer"].view(torch.int16))
    # rotations: bit-equal to the oracle (same fused-multiply-add placement)
    assert torch.equal(gpu["q"].cpu().contiguous().view(torch.int16), t["q"].contiguous().view(torch.int16))
    assert torch.equal(gpu["k"].cpu().contiguous().view(torch.int16), t["k"].contiguous().view(torch.int16))
    assert torch.equal(gpu["k_buffer"].cpu().view(torch.int16), t["k_buffer"].view(torch.int16))
    # and against an independent float64 rotation within bf16 rounding
    from oracle import build_ref

    ref = build_ref.load_rope()
    if ref is not None:
        t2 = _rope_inputs(spec["N"], spec["Hq"], spec["Hkv"], spec["D"], spec["rot"], 4096, 500, 3,
                          spec["pos"], spec["loc"], fused_qkv=spec.get("fused", True))
        g2 = _to_cuda(t2, spec["Hq"], spec["Hkv"], spec["D"])
        _run_rope(ref, g2, spec["D"], spec["neox"])
        torch.cuda.synchronize()
        assert torch.equal(g2["q_pre"], gpu["q_pre"]) and torch.equal(g2["v_buffer"], gpu["v_buffer"])
        _ulp_close(g2["q"].contiguous().cpu(), gpu["q"].contiguous().cpu())
        _ulp_close(g2["k_buffer"].cpu(), gpu["k_buffer"].cpu())


def test_rope_rotation_is_a_rotation():
    """Independent check in float64: norms of rotated pairs are preserved."""
    ext = load_mac_decode_rope_preserve_extension()
    t = _rope_inputs(16, 32, 8, 128, 128, 8192, 64, 9, torch.int64, torch.int64)
    gpu = _to_cuda(t, 32, 8, 128)
    q0 = t["q"].clone().double().view(16, 32, 128)
    _run_rope(ext, gpu, 128, True)
    torch.cuda.synchronize()
    q1 = gpu["q"].cpu().double().view(16, 32, 128)
    cs = t["cache"].double()[t["positions"].long()]
    c, s = cs[:, None, :64], cs[:, None, 64:]
    exp0 = q0[..., :64] * c - q0[..., 64:] * s
    exp1 = q0[..., 64:] * c + q0[..., :64] * s
    exp = torch.cat([exp0, exp1], dim=-1)
    assert (q1 - exp).abs().max() <= 0.02 * exp.abs().max()
    assert O.rel_l2(q1, exp) < 4e-3


def test_rope_argument_errors():
    ext = load_mac_decode_rope_preserve_extension()
    t = _to_cuda(_rope_inputs(4, 8, 2, 128, 128, 128, 32, 1, torch.int64, torch.int64), 8, 2, 128)
    with pytest.raises(RuntimeError, match="invalid head_dim"):
        ext.mac_decode_rope_preserve_q_bf16(t["q"], t["k"], t["v"], t["q_pre"], t["k_buffer"],
                                            t["v_buffer"], t["cache"], t["positions"], t["locs"],
                                            96, True)
    with pytest.raises(RuntimeError, match="wrong dtype"):
        ext.mac_decode_rope_preserve_q_bf16(t["q"].float(), t["k"], t["v"], t["q_pre"],
                                            t["k_buffer"], t["v_buffer"], t["cache"],
                                            t["positions"], t["locs"], 128, True)


def _downdate_inputs(N, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    out1 = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    out2 = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    lse1 = torch.randn(N, H, generator=g) * 2 + 6
    lse2 = lse1 - torch.rand(N, H, generator=g) * 5 - 0.01      # window mass < total mass
    lse2[0, 0] = lse1[0, 0]                                    # window == whole -> empty state
    if N > 1:
        lse2[1, 0] = lse1[1, 0] + 0.5                          # inconsistent -> keep (out1, lse1)
        lse2[1, 1] = -float("inf")                             # empty window
    return out1, lse1, out2, lse2


@pytest.mark.parametrize("N,H,D", [(300, 32, 128), (5, 3, 64), (9, 4, 40), (2, 2, 1024), (70, 5, 16),
                                   (33, 2, 8), (64, 4, 32)])
def test_downdate_matches_oracle_and_reference(N, H, D):
    ext = load_mac_merge_downdate_cache_extension()
    out1, lse1, out2, lse2 = _downdate_inputs(N, H, D, 5)
    c_out2, c_lse2 = out2.clone(), lse2.clone()
    O.update_then_downdate(out1, lse1, c_out2, c_lse2)
    g_out2, g_lse2 = out2.cuda(), lse2.cuda()
    ext.mac_update_then_downdate_bf16_inplace(out1.cuda(), lse1.cuda(), g_out2, g_lse2)
    torch.cuda.synchronize()
    fin = torch.isfinite(c_lse2)
    assert torch.equal(torch.isfinite(g_lse2.cpu()), fin)
    assert (g_lse2.cpu()[fin] - c_lse2[fin]).abs().max() <= 1e-4
    assert O.rel_l2(g_out2.float().cpu(), c_out2.float()) <= 2e-3
    # guard rows
    assert torch.equal(g_out2[0, 0].cpu(), torch.zeros(D, dtype=torch.bfloat16))
    if N > 1:
        assert torch.equal(g_out2[1, 0].cpu(), out1[1, 0]) and float(g_lse2[1, 0]) == float(lse1[1, 0])
        assert torch.equal(g_out2[1, 1].cpu(), out1[1, 1])
    from oracle import build_ref

    ref = build_ref.load_downdate()
    if ref is not None:
        r_out2, r_lse2 = out2.cuda(), lse2.cuda()
        ref.mac_update_then_downdate_bf16_inplace(out1.cuda(), lse1.cuda(), r_out2, r_lse2)
        torch.cuda.synchronize()
        assert torch.equal(torch.isfinite(r_lse2), torch.isfinite(g_lse2))
        m = torch.isfinite(r_lse2)
        assert (r_lse2[m] - g_lse2[m]).abs().max() <= 1e-3       # the reference uses fast-math exp/log
        assert O.rel_l2(g_out2.float().cpu(), r_out2.float().cpu()) <= 1e-2


@pytest.mark.parametrize("dt1,dt2", [(torch.float16, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.float16)])
def test_downdate_lse_element_types(dt1, dt2):
    ext = load_mac_merge_downdate_cache_extension()
    out1, lse1, out2, lse2 = _downdate_inputs(40, 8, 128, 7)
    l1, l2 = lse1.to(dt1), lse2.to(dt2)
    c_out2, c_lse2 = out2.clone(), l2.float().clone()
    O.update_then_downdate(out1, l1.float(), c_out2, c_lse2)
    g_out2, g_lse2 = out2.cuda(), l2.cuda()
    ext.mac_update_then_downdate_bf16_inplace(out1.cuda(), l1.cuda(), g_out2, g_lse2)
    torch.cuda.synchronize()
    assert g_lse2.dtype == dt2
    fin = torch.isfinite(c_lse2)
    assert torch.equal(torch.isfinite(g_lse2.float().cpu()), fin)
    assert (g_lse2.float().cpu()[fin] - c_lse2[fin]).abs().max() <= 0.07
    assert O.rel_l2(g_out2.float().cpu(), c_out2.float()) <= 2e-3


def test_downdate_then_merge_recovers_the_prefix_state():
    """Property: for attention states, (whole minus window) merged with the window
    gives back the whole."""
    ext = load_mac_merge_downdate_cache_extension()
    g = torch.Generator().manual_seed(2)
    T, H, D, S = 600, 8, 128, 64
    q = torch.randn(H, D, generator=g)
    k = torch.randn(T, D, generator=g)
    v = torch.randn(T, D, generator=g)

    def attn(lo, hi):
        s = (q @ k[lo:hi].T) / math.sqrt(D)
        lse = torch.logsumexp(s, dim=1)
        return (torch.softmax(s, dim=1) @ v[lo:hi]), lse

    o_all, l_all = attn(0, T)
    o_win, l_win = attn(T - S, T)
    o_pre, l_pre = attn(0, T - S)
    out1 = o_all.to(torch.bfloat16)[None].contiguous().cuda()
    out2 = o_win.to(torch.bfloat16)[None].contiguous().cuda()
    lse1, lse2 = l_all[None].contiguous().cuda(), l_win[None].contiguous().cuda()
    ext.mac_update_then_downdate_bf16_inplace(out1, lse1, out2, lse2)
    torch.cuda.synchronize()
    assert (lse2.cpu()[0] - l_pre).abs().max() < 2e-2
    assert O.rel_l2(out2.float().cpu()[0], o_pre) < 3e-2


@pytest.mark.parametrize("chunk", range(3))
def test_rope_preserve_random_matrix(chunk):
    """Seeded random shapes (head counts, head / rotary sizes incl. ones only the scalar path
    takes, both layouts, index types, fused or separate q/k/v) against the CPU oracle, bit for bit."""
    import random

    ext = load_mac_decode_rope_preserve_extension()
    rng = random.Random(40 + chunk)
    for i in range(12):
        Hkv = rng.choice([1, 2, 4, 8])
        Hq = Hkv * rng.choice([1, 2, 4, 8])
        D = rng.choice([16, 40, 64, 80, 128, 256])
        rot = rng.choice([D, D // 2, 8])
        rot -= rot % 2
        spec = dict(N=rng.randint(1, 70), Hq=Hq, Hkv=Hkv, D=D, rot=rot, neox=rng.random() < 0.5,
                    pos=rng.choice([torch.int32, torch.int64]),
                    loc=rng.choice([torch.int32, torch.int64]), fused=rng.random() < 0.7)
        t = _rope_inputs(spec["N"], Hq, Hkv, D, rot, 2048, 200, 100 * chunk + i, spec["pos"],
                         spec["loc"], fused_qkv=spec["fused"])
        gpu = _to_cuda(t, Hq, Hkv, D)
        q_before = t["q"].clone()
        O.decode_rope_preserve(t["q"], t["k"], t["v"], t["q_pre"], t["k_buffer"], t["v_buffer"],
                               t["cache"], t["positions"], t["locs"], D, spec["neox"])
        _run_rope(ext, gpu, D, spec["neox"])
        torch.cuda.synchronize()
        N = spec["N"]
        tag = f"chunk {chunk} case {i}: {spec}"
        assert torch.equal(gpu["q_pre"].cpu()[:N].view(N, -1).view(torch.int16),
                           q_before.contiguous().view(torch.int16)), tag
        for name in ("q", "k"):
            assert torch.equal(gpu[name].cpu().contiguous().view(torch.int16),
                               t[name].contiguous().view(torch.int16)), (name, tag)
        for name in ("k_buffer", "v_buffer"):
            assert torch.equal(gpu[name].cpu().view(torch.int16), t[name].view(torch.int16)), (name, tag)


@pytest.mark.parametrize("chunk", range(2))
def test_downdate_random_matrix(chunk):
    import random

    ext = load_mac_merge_downdate_cache_extension()
    rng = random.Random(90 + chunk)
    for i in range(15):
        N, H = rng.randint(1, 300), rng.choice([1, 2, 3, 8, 32])
        D = rng.choice([8, 16, 24, 32, 40, 64, 128, 256, 1024])
        g = torch.Generator().manual_seed(10 * chunk + i)
        out1 = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
        out2 = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
        lse1 = torch.randn(N, H, generator=g) + 4
        lse2 = lse1 - torch.rand(N, H, generator=g) * 5 - 0.02
        lse2[0, 0] = lse1[0, 0]
        if N > 1:
            lse2[1, 0] = lse1[1, 0] + 2
        c_out2, c_lse2 = out2.clone(), lse2.clone()
        O.update_then_downdate(out1, lse1, c_out2, c_lse2)
        g_out2, g_lse2 = out2.cuda(), lse2.cuda()
        ext.mac_update_then_downdate_bf16_inplace(out1.cuda(), lse1.cuda(), g_out2, g_lse2)
        torch.cuda.synchronize()
        tag = f"chunk {chunk} case {i}: N{N} H{H} D{D}"
        fin = torch.isfinite(c_lse2)
        assert torch.equal(torch.isfinite(g_lse2.cpu()), fin), tag
        assert torch.allclose(g_lse2.cpu()[fin], c_lse2[fin], rtol=1e-5, atol=1e-5), tag
        assert O.rel_l2(g_out2.float().cpu(), c_out2.float()) <= 2e-3, tag
