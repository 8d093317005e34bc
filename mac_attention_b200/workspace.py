"""The 30-tensor decode workspace, in the reference operator's argument order.

Shapes follow the reference's own callers (its tests, tools and SGLang hook all
build the same list, e.g. ``attention/tools/bench_mac_persistent_decode.py:15-58``)
and its launcher's lower bounds (``csrc/mac_decode_persistent.cu:5101-5153``).
This kernel only fills the decision arrays (indices 0-15), ``task_counts`` (22)
and ``phase_cycles`` (29); the task lists and partial buffers exist for
signature compatibility (their shapes are checked, their contents never touched).
"""
from __future__ import annotations

import torch

# indices into the returned list
HEAD_HIT, HEAD_MATCH_SLOT, HEAD_MATCH_POS = 3, 4, 5
HEAD_PREFIX_END, HEAD_RECT_START, HEAD_NEW_END = 6, 7, 8
GROUP_RECT_BEGIN, GROUP_MODE, TASK_COUNTS, PHASE_CYCLES = 9, 15, 22, 29


def make_decode_workspace(batch, hq, hkv, capacity, max_context, tile_tokens, match_tile_slots,
                          semantic_pos_ahead, front_sink_tokens=0, *, device="cuda",
                          partial_dtype=torch.float32, phase_slots=16):
    group = hq // hkv
    dim = 128
    tm = (capacity + match_tile_slots - 1) // match_tile_slots
    tc = (max_context + tile_tokens - 1) // tile_tokens
    tc += (max(front_sink_tokens, 0) + tile_tokens - 1) // tile_tokens
    tr = (tc + 31) // 32
    tt = max(1, (max(semantic_pos_ahead, 1) + tile_tokens - 1) // tile_tokens)
    i32 = dict(device=device, dtype=torch.int32)
    return [
        torch.empty(batch, hq, tm, device=device, dtype=torch.float32),
        torch.empty(batch, hq, tm, **i32),
        torch.empty(batch, hq, tm, **i32),
        *[torch.empty(batch, hq, **i32) for _ in range(6)],
        *[torch.empty(batch, hkv, **i32) for _ in range(6)],
        torch.empty(batch, hkv, **i32),
        torch.empty(batch * hq * tc, **i32),
        torch.empty(batch * hq * tc, **i32),
        torch.empty(batch * hkv * tt, **i32),
        torch.empty(batch * hkv * tt, **i32),
        torch.empty(batch * hq * tt, **i32),
        torch.empty(batch * hq * tt, **i32),
        torch.empty(9, **i32),
        torch.empty(batch, hkv, tc, group, dim, device=device, dtype=partial_dtype),
        torch.empty(batch, hkv, tc, group, device=device, dtype=torch.float32),
        torch.empty(batch, hkv, tr, group, dim, device=device, dtype=partial_dtype),
        torch.empty(batch, hkv, tr, group, device=device, dtype=torch.float32),
        torch.empty(batch, hkv, tt, group, dim, device=device, dtype=partial_dtype),
        torch.empty(batch, hkv, tt, group, device=device, dtype=torch.float32),
        torch.zeros(phase_slots, device=device, dtype=torch.int64),
    ]


def make_decision_workspace(batch, hq, hkv, capacity, match_tile_slots, *, device="cuda",
                            phase_slots=16):
    """The 18 observable workspace tensors only (a few hundred KB): the three
    per-tile match arrays, six per-head and seven per-group decision arrays,
    ``task_counts`` and ``phase_cycles`` -- what ``mac_persistent_decode_bf16_lean``
    takes instead of the reference's 30-tensor workspace."""
    tm = (capacity + match_tile_slots - 1) // match_tile_slots
    i32 = dict(device=device, dtype=torch.int32)
    return [
        torch.empty(batch, hq, tm, device=device, dtype=torch.float32),
        torch.empty(batch, hq, tm, **i32),
        torch.empty(batch, hq, tm, **i32),
        *[torch.empty(batch, hq, **i32) for _ in range(6)],
        *[torch.empty(batch, hkv, **i32) for _ in range(7)],
        torch.empty(9, **i32),
        torch.zeros(phase_slots, device=device, dtype=torch.int64),
    ]
