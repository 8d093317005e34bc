"""Synthetic chunked-prefill inputs for the ring-build tests: prompts with real
attention states (full prefix, trailing window) computed in float64, and the
state a ring row must hold under a front sink, computed directly."""
import math

import torch

from mac_attention_b200 import ops


def attention_state(scores, v, mask):
    """Softmax state of masked scores: scores [H,n,T] f64, v [H,T,D] f64, mask [n,T] bool."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                         # [H,n]
    w = torch.exp(s - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None])
    w = torch.where(mask[None], w, torch.zeros_like(w))
    return torch.einsum("hnt,htd->nhd", w, v), lse.transpose(0, 1).contiguous()   # [n,H,D], [n,H]


def make_prompts(lens, L0s, Hq, Hkv, S, F, M, seed, max_ctx=2048, sink_gain=1.5):
    """Chunked-prefill inputs of requests with L0 cached tokens and ``len`` new ones."""
    D = 128
    g = torch.Generator().manual_seed(seed)
    B, G = len(lens), Hq // Hkv
    totals = [a + b for a, b in zip(L0s, lens)]
    pool_rows = sum(totals) + 64 + B
    perm = torch.randperm(pool_rows, generator=g)
    k = torch.randn(pool_rows, Hkv, D, generator=g)
    v = torch.randn(pool_rows, Hkv, D, generator=g)
    req_to_token = torch.zeros(B, max_ctx, dtype=torch.int32)
    at = 0
    for b, t in enumerate(totals):
        req_to_token[b, :t + 1] = perm[at:at + t + 1].to(torch.int32)   # one spare slot for a decode token
        at += t + 1
        k[req_to_token[b, :F].long()] *= sink_gain                      # heavy sink keys
    k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)
    rows = sum(lens)
    q_post = torch.randn(rows, Hq, D, generator=g).to(torch.bfloat16)
    q_pre = torch.randn(rows, Hq, D, generator=g).to(torch.bfloat16)
    full_o, full_l, band_o, band_l = [], [], [], []
    want_o, want_l = [], []
    scale = 1.0 / math.sqrt(D)
    off = 0
    for b in range(B):
        T, n, L0 = totals[b], lens[b], L0s[b]
        tok = req_to_token[b, :T].long()
        kk = k[tok].double().repeat_interleave(G, dim=1).permute(1, 0, 2)   # [H,T,D]
        vv = v[tok].double().repeat_interleave(G, dim=1).permute(1, 0, 2)
        q = q_post[off:off + n].double().permute(1, 0, 2)                   # [H,n,D]
        sc = torch.einsum("hnd,htd->hnt", q, kk) * scale
        pos = torch.arange(L0, L0 + n)[:, None]
        t = torch.arange(T)[None]
        E = (pos + 1 - S).clamp(min=0)
        o, l = attention_state(sc, vv, t <= pos)
        full_o.append(o), full_l.append(l)
        o, l = attention_state(sc, vv, (t >= E) & (t <= pos))
        band_o.append(o), band_l.append(l)
        o, l = attention_state(sc, vv, (t >= torch.minimum(E, torch.tensor(F))) & (t < E))
        want_o.append(o), want_l.append(l)
        off += n
    offsets = torch.zeros(B + 1, dtype=torch.int32)
    offsets[1:] = torch.tensor(lens).cumsum(0)
    R = B
    return dict(
        k=k, v=v, req_to_token=req_to_token, q_post=q_post, src_q=q_pre,
        full_attn=torch.cat(full_o).to(torch.bfloat16), full_lse=torch.cat(full_l).float(),
        band_attn=torch.cat(band_o).to(torch.bfloat16), band_lse=torch.cat(band_l).float(),
        want_o=torch.cat(want_o), want_l=torch.cat(want_l),
        offsets=offsets, lens=torch.tensor(lens, dtype=torch.int32),
        req_ids=torch.arange(B, dtype=torch.int32),
        request_length=torch.tensor(L0s, dtype=torch.int32),
        q_cache=torch.zeros(R, M, Hq, D, dtype=torch.bfloat16),
        attn_cache=torch.full((R, M, Hq, D), 7.0, dtype=torch.bfloat16),
        lse_cache=torch.full((R, M, Hq), 3.0),
        q_post_cache=torch.zeros(R, M, Hq, D, dtype=torch.bfloat16),
        ready=torch.zeros(R, dtype=torch.bool), cache_epoch=torch.full((R,), -1, dtype=torch.int64),
        request_epoch=torch.arange(R, dtype=torch.int64) + 2,
    )


def run_build(mod_fn, t, M, Hq, S, F):
    mod_fn(t["q_cache"], t["attn_cache"], t["lse_cache"], t["request_length"], t["req_ids"],
           t["src_q"], t["full_attn"], t["full_lse"], t["band_attn"], t["band_lse"], t["offsets"],
           t["lens"], M, Hq, 128, t["q_post_cache"], sink_mode=ops.SINK_EXCLUDE, ready=t["ready"],
           cache_epoch=t["cache_epoch"], request_epoch=t["request_epoch"], q_post=t["q_post"],
           k_buffer=t["k"], v_buffer=t["v"], req_to_token=t["req_to_token"], front_sink_tokens=F,
           semantic_pos_ahead=S)


SPECS = [
    dict(lens=[200, 37, 300], L0s=[0, 150, 90], Hq=8, Hkv=2, S=16, F=64, M=256),
    dict(lens=[330, 270], L0s=[0, 20], Hq=8, Hkv=1, S=8, F=128, M=64),      # G=8, ring wraps, start > 0
    dict(lens=[90], L0s=[40], Hq=4, Hkv=4, S=4, F=20, M=128),               # G=1, F not a multiple of 16
    dict(lens=[50, 60], L0s=[0, 0], Hq=32, Hkv=2, S=16, F=16, M=128),       # G=16
]
