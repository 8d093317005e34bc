"""Shared plumbing of the parity tests: run one decode step through the CUDA
operator (C ABI) or through the CPU oracle on the same inputs and compare."""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch

from mac_attention_b200 import load_mac_persistent_decode_extension, make_decode_workspace
from mac_attention_b200.synth import DecodeCase
from oracle import mac_oracle as O

REL_L2_TOL = 1e-2  # the reference's stated output tolerance vs its FP32 oracle


def case_from_golden(g) -> DecodeCase:
    i = g["inputs"]
    return DecodeCase(q_post=i["q_post"], q_pre=i["q_pre"], k=i["k"], v=i["v"],
                      req_to_token=i["req_to_token"], req_ids=i["req_ids"],
                      past_lens=i["past_lens"], out_cache_loc=i["out_cache_loc"],
                      query_cache=i["query_cache"].clone(), attn_cache=i["attn_cache"].clone(),
                      lse_cache=i["lse_cache"].clone())


def run_oracle(case: DecodeCase, cfg: O.DecodeConfig):
    """CPU oracle on a CPU copy of the case; returns (result, ring tensors after the step)."""
    c = case.to("cpu").clone()
    res = O.decode_step(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens,
                        c.out_cache_loc, c.query_cache, c.attn_cache, c.lse_cache, cfg,
                        c.cache_ready, c.cache_epoch, c.request_epoch)
    return res, c


def run_cuda(case: DecodeCase, cfg: O.DecodeConfig, *, ws_batch=None, ext=None,
             partial_dtype=torch.float32, workspace=None, poison=True):
    """CUDA operator on a CUDA copy of the case (ring tensors updated in place on the copy)."""
    ext = ext or load_mac_persistent_decode_extension()
    c = case.to("cuda").clone()
    N, Hq, D = c.q_post.shape
    Hkv = c.k.shape[1]
    M = c.query_cache.shape[1]
    ws = workspace or make_decode_workspace(ws_batch or N, Hq, Hkv, M, cfg.max_context,
                                            cfg.tile_tokens, cfg.match_tile_slots,
                                            cfg.semantic_pos_ahead, cfg.front_sink_tokens,
                                            partial_dtype=partial_dtype)
    if poison and workspace is None:
        for t in ws[:22]:
            t.fill_(-7 if t.dtype != torch.float32 else float("nan"))
    out = torch.full_like(c.q_post, float("nan"))
    lse = torch.full((N, Hq), float("nan"), device="cuda")
    empty = torch.empty(0)
    ext.mac_persistent_decode_bf16(
        c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens, c.out_cache_loc,
        c.query_cache, c.attn_cache, c.lse_cache, out, lse, *ws, *cfg.scalar_args(),
        c.query_cache,
        c.cache_ready if c.cache_ready is not None else empty,
        c.cache_epoch if c.cache_epoch is not None else empty,
        c.request_epoch if c.request_epoch is not None else empty)
    torch.cuda.synchronize()
    return SimpleNamespace(out=out, lse=lse, ws=ws, case=c)


def ring_rows(case: DecodeCase):
    """Ring row written this step per batch row: (q, o, lse) at slot P mod M."""
    M = case.query_cache.shape[1]
    qs, os_, ls = [], [], []
    for n in range(case.q_post.shape[0]):
        req, P = int(case.req_ids[n]), int(case.past_lens[n])
        qs.append(case.query_cache[req, P % M])
        os_.append(case.attn_cache[req, P % M])
        ls.append(case.lse_cache[req, P % M])
    return torch.stack(qs), torch.stack(os_), torch.stack(ls)


def assert_decisions_equal(cu, orc, N):
    ws = cu.ws
    pairs = [(3, orc.head_hit, "head_hit"), (4, orc.head_match_slot, "head_match_slot"),
             (5, orc.head_match_pos, "head_match_pos"), (6, orc.head_prefix_end, "head_prefix_end"),
             (7, orc.head_rect_start, "head_rect_start"), (8, orc.head_new_end, "head_new_end"),
             (9, orc.group_rect_begin, "group_rect_begin"), (15, orc.group_mode, "group_mode")]
    for idx, ref, name in pairs:
        got = ws[idx][:N].cpu()
        assert torch.equal(got, ref), f"{name} differs: {got.flatten()[:32]} vs {ref.flatten()[:32]}"
    tc = ws[22].cpu()
    assert int(tc[5]) == int(orc.task_counts[5]) and int(tc[6]) == int(orc.task_counts[6])


def assert_outputs_close(cu, orc, orc_case, tol=REL_L2_TOL, ready_rows=None):
    """rel-L2 of output, ring state and LSEs against the oracle (per tensor)."""
    out = cu.out.float().cpu()
    assert torch.isfinite(out).all()
    assert O.rel_l2(out, orc.out_f32) <= tol, f"out rel_l2 {O.rel_l2(out, orc.out_f32)}"
    lse_c, lse_o = cu.lse.cpu(), orc.lse
    fin = torch.isfinite(lse_o)
    assert torch.equal(torch.isfinite(lse_c), fin)
    assert (lse_c[fin] - lse_o[fin]).abs().max() <= 2e-2 if fin.any() else True
    q_c, o_c, l_c = ring_rows(cu.case.to("cpu"))
    q_o, o_o, l_o = ring_rows(orc_case)
    assert torch.equal(q_c, q_o), "ring query rows differ"
    assert O.rel_l2(o_c.float(), o_o.float()) <= tol, "ring state rows differ"
    fin = torch.isfinite(l_o)
    assert torch.equal(torch.isfinite(l_c), fin)
    if fin.any():
        assert (l_c[fin] - l_o[fin]).abs().max() <= 2e-2
