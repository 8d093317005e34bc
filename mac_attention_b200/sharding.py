"""KV-head sharding of a decode step across GPUs (tensor parallel).

Every quantity of the path is indexed by (request, KV head) and heads of
different KV groups never interact, so rank ``r`` of ``W`` owns KV heads
``[r*Hkv/W, (r+1)*Hkv/W)`` with the matching query heads, its own slice of the
KV pool, of the ring and of the workspace, and runs an ordinary decode step on
it.  No data crosses ranks inside attention (the reference relies on SGLang
handing it per-rank head counts, ``llama_hooks.py:1058-1061`` in the reference
project); the model's output projection all-reduce lives outside this path.
"""
from __future__ import annotations

import torch

from .synth import DecodeCase


def head_slices(hq: int, hkv: int, world_size: int, rank: int):
    if hkv % world_size != 0:
        raise ValueError(f"Hkv={hkv} is not divisible by world size {world_size}")
    g = hq // hkv
    kv_per = hkv // world_size
    kv = slice(rank * kv_per, (rank + 1) * kv_per)
    q = slice(rank * kv_per * g, (rank + 1) * kv_per * g)
    return q, kv


def shard_case(case: DecodeCase, world_size: int, rank: int) -> DecodeCase:
    """The rank's own contiguous copy of every head-indexed tensor."""
    hq, hkv = case.q_post.shape[1], case.k.shape[1]
    q, kv = head_slices(hq, hkv, world_size, rank)
    out = case.clone()
    out.q_post = case.q_post[:, q].contiguous()
    out.q_pre = case.q_pre[:, q].contiguous()
    out.k = case.k[:, kv].contiguous()
    out.v = case.v[:, kv].contiguous()
    out.query_cache = case.query_cache[:, :, q].contiguous()
    out.attn_cache = case.attn_cache[:, :, q].contiguous()
    out.lse_cache = case.lse_cache[:, :, q].contiguous()
    out.meta = dict(case.meta, rank=rank, world_size=world_size)
    return out


def gather_heads(parts: list[torch.Tensor], dim: int = 1) -> torch.Tensor:
    """Concatenate per-rank head slices back in rank order."""
    return torch.cat(parts, dim=dim)
