"""Seeded synthetic decode steps with the shapes and value distributions of the
reference's benchmarks (``attention/tools/bench_mac_persistent_decode.py:61-113``
in the reference project builds the same kind of case on the device).

The reference measures on synthetic tensors only; these generators stand in
for serving traces: K/V ~ N(0, sigma_kv), queries ~ N(0, 1), a ring whose rows
are either far from the query (``N(0,1) + 10``), planted near-duplicates
(``q + N(0, noise)``, a hit) or borderline rows whose distance sits next to the
threshold.  KV pools are paged: ``page_size`` consecutive logical positions
share a page and pages are scattered over the pool by a seeded permutation,
while ``req_to_token`` stays a per-token table as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class DecodeCase:
    q_post: torch.Tensor
    q_pre: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    req_to_token: torch.Tensor
    req_ids: torch.Tensor
    past_lens: torch.Tensor
    out_cache_loc: torch.Tensor
    query_cache: torch.Tensor
    attn_cache: torch.Tensor
    lse_cache: torch.Tensor
    cache_ready: torch.Tensor | None = None
    cache_epoch: torch.Tensor | None = None
    request_epoch: torch.Tensor | None = None
    meta: dict = field(default_factory=dict)

    def tensors(self):
        return {k: v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor)}

    def to(self, device):
        kw = {k: (v.to(device) if isinstance(v, torch.Tensor) else v)
              for k, v in self.__dict__.items()}
        return DecodeCase(**kw)

    def clone(self):
        kw = {k: (v.clone() if isinstance(v, torch.Tensor) else v)
              for k, v in self.__dict__.items()}
        kw["meta"] = dict(self.meta)
        return DecodeCase(**kw)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn_bf16(shape, gen, device, scale=1.0, shift=0.0, chunk_rows=1 << 16):
    """bf16 normal tensor, drawn in row chunks so the fp32 staging stays small."""
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    flat = out.view(shape[0], -1)
    for r0 in range(0, shape[0], chunk_rows):
        r1 = min(shape[0], r0 + chunk_rows)
        t = torch.randn(r1 - r0, flat.shape[1], generator=gen, device=device)
        if scale != 1.0:
            t.mul_(scale)
        if shift != 0.0:
            t.add_(shift)
        flat[r0:r1] = t.to(torch.bfloat16)
    return out


def make_decode_case(*, batch, ctx, hq=32, hkv=8, capacity=2048, page_size=16, seed=0,
                     device="cpu", kv_scale=1.0, ring_rows=None, ctx_list=None,
                     loc_dtype=torch.int32, sink_boost=0, shuffle_pages=True,
                     req_ids=None) -> DecodeCase:
    """A decode step over ``batch`` requests with ``ctx`` past tokens each
    (``ctx_list`` overrides per request).  The ring holds far rows only; use the
    ``plant_*`` helpers to add matches.  ``req_ids`` (default ``0..batch-1``)
    are the request-pool rows the batch rows live in; they index both
    ``req_to_token`` and the ring, so both get ``ring_rows`` rows."""
    dim = 128
    dev = torch.device(device)
    ctxs = [int(c) for c in (ctx_list if ctx_list is not None else [ctx] * batch)]
    assert len(ctxs) == batch
    kv_lens = [c + 1 for c in ctxs]
    pages = [(n + page_size - 1) // page_size for n in kv_lens]
    total_pages = sum(pages)
    pool_tokens = total_pages * page_size
    g = _gen(seed, dev)
    k = _randn_bf16((pool_tokens, hkv, dim), g, dev, scale=kv_scale)
    v = _randn_bf16((pool_tokens, hkv, dim), g, dev, scale=kv_scale)
    q_pre = _randn_bf16((batch, hq, dim), g, dev)
    q_post = _randn_bf16((batch, hq, dim), g, dev)
    stride = max(kv_lens)
    gcpu = _gen(seed + 1, "cpu")
    perm = torch.randperm(total_pages, generator=gcpu) if shuffle_pages else torch.arange(total_pages)
    rids = [int(r) for r in (req_ids if req_ids is not None else range(batch))]
    R = ring_rows if ring_rows is not None else max(rids) + 1
    assert len(rids) == batch and max(rids) < R and len(set(rids)) == batch
    r2t = torch.zeros(R, stride, dtype=torch.int32)
    ocl = torch.zeros(batch, dtype=loc_dtype)
    p0 = 0
    offs = torch.arange(page_size, dtype=torch.int64)
    for n in range(batch):
        pg = perm[p0:p0 + pages[n]].to(torch.int64)
        p0 += pages[n]
        toks = (pg[:, None] * page_size + offs[None, :]).reshape(-1)[:kv_lens[n]]
        r2t[rids[n], :ctxs[n]] = toks[:ctxs[n]].to(torch.int32)
        ocl[n] = int(toks[ctxs[n]])
    if sink_boost > 0:
        # sink-heavy softmax mass: keys of the first positions are scaled x4
        for n in range(batch):
            rows = r2t[rids[n], :min(sink_boost, ctxs[n])].to(torch.int64).to(dev)
            k[rows] = (k[rows].float() * 4).to(torch.bfloat16)
    qc = _randn_bf16((R * capacity, hq, dim), g, dev, shift=10.0).view(R, capacity, hq, dim)
    ac = torch.zeros_like(qc)
    lc = torch.zeros(R, capacity, hq, dtype=torch.float32, device=dev)
    return DecodeCase(
        q_post=q_post, q_pre=q_pre, k=k, v=v, req_to_token=r2t.to(dev),
        req_ids=torch.tensor(rids, dtype=torch.int32, device=dev),
        past_lens=torch.tensor(ctxs, dtype=torch.int32, device=dev),
        out_cache_loc=ocl.to(dev), query_cache=qc, attn_cache=ac, lse_cache=lc,
        meta=dict(batch=batch, hq=hq, hkv=hkv, capacity=capacity, page_size=page_size,
                  seed=seed, ctxs=ctxs))


def ring_slot(past_len: int, capacity: int, pos: int) -> int:
    """Ring slot holding logical position ``pos`` (``pos mod capacity``)."""
    return pos % capacity


def plant_matches(case: DecodeCase, *, hit_fraction: float, noise: float = 0.1, lag_lo: int = 1,
                  lag_hi: int | None = None, seed: int = 0, borderline_fraction: float = 0.0,
                  threshold: float = 0.45, state_scale: float = 1.0,
                  heads_per_draw: int = 1) -> torch.Tensor:
    """Plant ring entries so that about ``hit_fraction`` of the (request, head)
    pairs find a near-duplicate of their pre-RoPE query at a position drawn
    uniformly from ``[P - lag_hi, P - lag_lo]``.  Planted rows get a finite
    prefix state (random o, finite LSE).  ``borderline_fraction`` of the other
    pairs get a row whose squared distance sits within ~1% of the threshold, on
    either side.  ``heads_per_draw`` > 1 draws hit/miss once per that many
    consecutive heads (one KV group), the way the reference's synthetic benchmark
    mode clusters its misses.  Returns the bool mask [batch, hq] of planted hits."""
    g = _gen(seed + 77, "cpu")
    batch, hq, dim = case.q_pre.shape
    cap = case.query_cache.shape[1]
    dev = case.q_pre.device
    thr = 2.0 * dim * (1.0 - threshold) ** 2
    planted = torch.zeros(batch, hq, dtype=torch.bool)
    for n in range(batch):
        P = int(case.past_lens[n])
        req = int(case.req_ids[n])
        max_lag = min(cap, P)
        if max_lag < 1:
            continue
        hi = min(lag_hi if lag_hi is not None else max_lag, max_lag)
        lo = min(max(lag_lo, 1), hi)
        u = torch.rand(hq, generator=g)
        if heads_per_draw > 1:
            u = u[::heads_per_draw].repeat_interleave(heads_per_draw)[:hq]
        lag = torch.randint(lo, hi + 1, (hq,), generator=g)
        ub = torch.rand(hq, generator=g)
        for h in range(hq):
            pos = P - int(lag[h])
            slot = ring_slot(P, cap, pos)
            q = case.q_pre[n, h].float().cpu()
            if u[h] < hit_fraction:
                row = q + noise * torch.randn(dim, generator=g)
                planted[n, h] = True
            elif ub[h] < borderline_fraction:
                # distance = thr * (1 +- ~1%): exercises the exact summation order
                d = torch.randn(dim, generator=g)
                tgt = thr * (1.0 + 0.01 * (2 * float(torch.rand((), generator=g)) - 1))
                row = q + d * math.sqrt(tgt / float((d * d).sum()))
            else:
                continue
            case.query_cache[req, slot, h] = row.to(torch.bfloat16).to(dev)
            case.attn_cache[req, slot, h] = (state_scale * torch.randn(dim, generator=g)).to(
                torch.bfloat16).to(dev)
            case.lse_cache[req, slot, h] = float(torch.randn((), generator=g)) + 5.0
    return planted


def add_readiness_gate(case: DecodeCase, *, not_ready_fraction=0.2, stale_fraction=0.1, seed=0):
    """Readiness tensors: some requests not ready, some with a stale cache epoch."""
    g = _gen(seed + 991, "cpu")
    R = case.query_cache.shape[0]
    dev = case.q_pre.device
    u = torch.rand(R, generator=g)
    ready = u >= not_ready_fraction
    request_epoch = torch.randint(0, 5, (R,), generator=g, dtype=torch.int64)
    cache_epoch = request_epoch.clone()
    stale = (u >= not_ready_fraction) & (u < not_ready_fraction + stale_fraction)
    cache_epoch[stale] -= 1
    case.cache_ready = ready.to(dev)
    case.cache_epoch = cache_epoch.to(dev)
    case.request_epoch = request_epoch.to(dev)
    case.meta["gated_off"] = (~ready | stale)
    return case
