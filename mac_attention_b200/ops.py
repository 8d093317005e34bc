"""Operators with the reference extension modules' names and positional signatures.

``mac_persistent_decode_bf16`` takes the 68 positional arguments of the
reference operator (``csrc/mac_decode_persistent.cu:4962-5030`` in the reference
project), ``mac_prefill_update_cache`` and the three gate/state operators take
those of ``csrc/mac_prefill_update_cache.cu:324-337, 374-495``.  Each one checks
what the reference launcher checks (same messages, ``RuntimeError``), fills the
plain-C argument struct and calls the C ABI on torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _abi

_BF16, _F32, _I32, _I64 = torch.bfloat16, torch.float32, torch.int32, torch.int64


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check(t: torch.Tensor, name: str, dtype: torch.dtype, dim: int) -> None:
    _req(t.is_cuda, f"{name} must be CUDA")
    _req(t.is_contiguous(), f"{name} must be contiguous")
    _req(t.dtype == dtype, f"{name} has wrong dtype")
    _req(t.dim() == dim, f"{name} has wrong rank")


def _check_partial_o(t: torch.Tensor, name: str) -> None:
    _req(t.is_cuda, f"{name} must be CUDA")
    _req(t.is_contiguous(), f"{name} must be contiguous")
    _req(t.dtype in (_F32, _BF16), f"{name} must be float32 or bfloat16")
    _req(t.dim() == 5, f"{name} has wrong rank")


def _env_flag(name: str, default: int) -> int:
    raw = os.environ.get(name)
    if raw is None:
        return default
    try:
        return 1 if int(raw) != 0 else 0
    except ValueError:
        return 0


def _env_int(name: str, default: int) -> int:
    raw = os.environ.get(name)
    if raw is None:
        return default
    try:
        v = int(raw)
    except ValueError:
        return default
    return v if v > 0 else default


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _decode_call(
    entry_name,
    q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids, past_lens, out_cache_loc,
    query_cache, attn_cache, lse_cache, out, optional_lse,
    match_dist, match_pos, match_slot,
    head_hit, head_match_slot, head_match_pos, head_prefix_end, head_rect_start, head_new_end,
    group_rect_begin, group_rect_end, group_rect_tiles,
    group_tail_begin, group_tail_end, group_tail_tiles, group_mode,
    complete_task_go, complete_task_tile, tail_task_go, tail_task_tile,
    hit_tail_task_ho, hit_tail_task_tile, task_counts,
    partial_rect_o, partial_rect_lse, partial_rect_reduced_o, partial_rect_reduced_lse,
    partial_tail_o, partial_tail_lse, phase_cycles,
    max_context, tile_tokens, match_tile_slots, semantic_pos_ahead, front_sink_tokens,
    gen_min_limit, lookback_right, candidate_mode, threshold, sm_scale,
    debug_enabled, bench_mode, bench_hit_rate, bench_hit_rate_std,
    bench_skip_ratio, bench_skip_ratio_std, bench_match_lag_mean, bench_match_lag_std,
    bench_seed, bench_miss_mask, bench_layer_id,
    query_post_cache, mac_cache_ready, mac_cache_epoch, mac_request_epoch,
) -> None:
    """Checks and argument marshalling shared by the decode entry points; returns the
    filled ``MacB200DecodeArgs``."""
    _check(q_post, "q_post", _BF16, 3)
    _check(q_pre, "q_pre", _BF16, 3)
    _check(k_buffer, "k_buffer", _BF16, 3)
    _check(v_buffer, "v_buffer", _BF16, 3)
    _check(req_to_token, "req_to_token", _I32, 2)
    _check(req_ids, "req_ids", _I32, 1)
    _check(past_lens, "past_lens", _I32, 1)
    _req(out_cache_loc.is_cuda, "out_cache_loc must be CUDA")
    _req(out_cache_loc.is_contiguous(), "out_cache_loc must be contiguous")
    _req(out_cache_loc.dim() == 1, "out_cache_loc has wrong rank")
    _req(out_cache_loc.dtype in (_I32, _I64), "out_cache_loc must be int32 or int64")
    _check(query_cache, "query_cache", _BF16, 4)
    if query_post_cache is not None and query_post_cache.numel() > 0:
        _check(query_post_cache, "query_post_cache", _BF16, 4)  # accepted, ignored
    _check(attn_cache, "attn_cache", _BF16, 4)
    _check(lse_cache, "lse_cache", _F32, 3)
    _check(out, "out", _BF16, 3)
    _req(optional_lse.is_cuda, "optional_lse must be CUDA")
    _req(optional_lse.is_contiguous(), "optional_lse must be contiguous")
    _req(optional_lse.numel() == 0 or optional_lse.dtype == _F32,
         "optional_lse must be empty or float32")
    _req(phase_cycles.is_cuda, "phase_cycles must be CUDA")
    _req(phase_cycles.is_contiguous(), "phase_cycles must be contiguous")
    _req(phase_cycles.dtype == _I64, "phase_cycles must be int64")
    _req(phase_cycles.numel() >= 6, "phase_cycles must have at least 6 elements")
    _check(match_dist, "match_dist", _F32, 3)
    _check(match_pos, "match_pos", _I32, 3)
    _check(match_slot, "match_slot", _I32, 3)
    for name, t in (("head_hit", head_hit), ("head_match_slot", head_match_slot),
                    ("head_match_pos", head_match_pos), ("head_prefix_end", head_prefix_end),
                    ("head_rect_start", head_rect_start), ("head_new_end", head_new_end),
                    ("group_rect_begin", group_rect_begin), ("group_rect_end", group_rect_end),
                    ("group_rect_tiles", group_rect_tiles), ("group_tail_begin", group_tail_begin),
                    ("group_tail_end", group_tail_end), ("group_tail_tiles", group_tail_tiles),
                    ("group_mode", group_mode)):
        _check(t, name, _I32, 2)
    lean = partial_rect_o is None   # the lean operator passes no task lists / partial buffers
    _check(task_counts, "task_counts", _I32, 1)
    if not lean:
        for name, t in (("complete_task_go", complete_task_go),
                        ("complete_task_tile", complete_task_tile),
                        ("tail_task_go", tail_task_go), ("tail_task_tile", tail_task_tile),
                        ("hit_tail_task_ho", hit_tail_task_ho),
                        ("hit_tail_task_tile", hit_tail_task_tile)):
            _check(t, name, _I32, 1)
        _check_partial_o(partial_rect_o, "partial_rect_o")
        _check(partial_rect_lse, "partial_rect_lse", _F32, 4)
        _check_partial_o(partial_rect_reduced_o, "partial_rect_reduced_o")
        _check(partial_rect_reduced_lse, "partial_rect_reduced_lse", _F32, 4)
        _check_partial_o(partial_tail_o, "partial_tail_o")
        _check(partial_tail_lse, "partial_tail_lse", _F32, 4)
        _req(partial_rect_reduced_o.dtype == partial_rect_o.dtype
             and partial_tail_o.dtype == partial_rect_o.dtype,
             "all partial output workspaces must use the same dtype")

    N, Hq, D = q_post.shape
    Hkv = k_buffer.shape[1]
    _req(D == 128, "persistent decode v1 supports D=128 only")
    _req(q_pre.shape == q_post.shape, "q_pre/q_post shape mismatch")
    _req(v_buffer.shape == k_buffer.shape, "k/v shape mismatch")
    _req(Hkv > 0 and Hq % Hkv == 0, "Hq must be divisible by Hkv")
    G = Hq // Hkv
    _req(0 < G <= 8, "unsupported GQA group size")
    _req(req_ids.shape[0] >= N and past_lens.shape[0] >= N and out_cache_loc.shape[0] >= N,
         "batch metadata too small")
    _req(out.shape == q_post.shape, "out shape mismatch")
    R, M = query_cache.shape[0], query_cache.shape[1]
    _req(query_cache.shape[2] == Hq and query_cache.shape[3] == D, "query_cache shape mismatch")
    _req(attn_cache.shape == query_cache.shape, "attn_cache shape mismatch")
    _req(tuple(lse_cache.shape) == (R, M, Hq), "lse_cache shape mismatch")

    tile_tokens = int(tile_tokens)
    match_tile_slots = int(match_tile_slots)
    max_context = int(max_context)
    Tm = match_dist.shape[2]
    _req(Tm >= (M + match_tile_slots - 1) // match_tile_slots, "match workspace too small")
    _req(group_mode.shape[0] >= N and group_mode.shape[1] >= Hkv, "group_mode workspace too small")
    _req(task_counts.numel() >= 9, "task_counts must have at least nine elements")
    _req(int(bench_mode) in (0, 1, 2), "unsupported synthetic MAC bench mode")
    if not lean:
        Tc = partial_rect_lse.shape[2]
        Tr = partial_rect_reduced_lse.shape[2]
        Tt = partial_tail_lse.shape[2]
        _req(Tm >= (M + match_tile_slots - 1) // match_tile_slots, "match workspace too small")
        _req(Tc >= (max_context + tile_tokens - 1) // tile_tokens, "rect workspace too small")
        _req(Tr >= (max_context + tile_tokens * 32 - 1) // (tile_tokens * 32),
             "reduced rect workspace too small")
        _req(Tt >= (int(semantic_pos_ahead) + tile_tokens - 1) // tile_tokens,
             "tail workspace too small")
        _req(partial_rect_o.shape[0] >= N and tuple(partial_rect_o.shape[1:]) == (Hkv, Tc, G, D),
             "rect output workspace has wrong shape")
        _req(partial_rect_lse.shape[0] >= N and tuple(partial_rect_lse.shape[1:]) == (Hkv, Tc, G),
             "rect lse workspace has wrong shape")
        _req(partial_rect_reduced_o.shape[0] >= N
             and tuple(partial_rect_reduced_o.shape[1:]) == (Hkv, Tr, G, D),
             "reduced rect output workspace has wrong shape")
        _req(partial_rect_reduced_lse.shape[0] >= N
             and tuple(partial_rect_reduced_lse.shape[1:]) == (Hkv, Tr, G),
             "reduced rect lse workspace has wrong shape")
        _req(partial_tail_o.shape[0] >= N and tuple(partial_tail_o.shape[1:]) == (Hkv, Tt, G, D),
             "tail output workspace has wrong shape")
        _req(partial_tail_lse.shape[0] >= N and tuple(partial_tail_lse.shape[1:]) == (Hkv, Tt, G),
             "tail lse workspace has wrong shape")
        _req(group_mode.shape[0] >= N and group_mode.shape[1] >= Hkv, "group_mode workspace too small")
        _req(complete_task_tile.numel() == complete_task_go.numel(), "complete task shape mismatch")
        _req(tail_task_tile.numel() == tail_task_go.numel(), "tail task shape mismatch")
        _req(hit_tail_task_tile.numel() == hit_tail_task_ho.numel(), "hit tail task shape mismatch")
        _req(task_counts.numel() >= 9, "task_counts must have at least nine elements")
        _req(int(bench_mode) in (0, 1, 2), "unsupported synthetic MAC bench mode")
        _req(complete_task_go.numel() >= N * Hq * Tc, "complete task workspace too small")
        _req(tail_task_go.numel() >= N * Hkv * Tt, "tail task workspace too small")
        _req(hit_tail_task_ho.numel() >= N * Hq * Tt, "hit tail task workspace too small")
    ws_batch = match_dist.shape[0]
    for name, t in (("match_dist", match_dist), ("match_pos", match_pos),
                    ("match_slot", match_slot)):
        _req(t.shape[0] >= N and t.shape[1] == Hq and t.shape[2] == Tm,
             f"{name} workspace has wrong shape")
    for name, t in (("head_hit", head_hit), ("head_match_slot", head_match_slot),
                    ("head_match_pos", head_match_pos), ("head_prefix_end", head_prefix_end),
                    ("head_rect_start", head_rect_start), ("head_new_end", head_new_end)):
        _req(t.shape[0] >= N and t.shape[1] == Hq, f"{name} workspace has wrong shape")
        ws_batch = min(ws_batch, t.shape[0])
    for name, t in (("group_rect_begin", group_rect_begin), ("group_rect_end", group_rect_end),
                    ("group_rect_tiles", group_rect_tiles), ("group_tail_begin", group_tail_begin),
                    ("group_tail_end", group_tail_end), ("group_tail_tiles", group_tail_tiles),
                    ("group_mode", group_mode)):
        _req(t.shape[0] >= N and t.shape[1] == Hkv, f"{name} workspace has wrong shape")
        ws_batch = min(ws_batch, t.shape[0])

    ready_ptr = epoch_ptr = req_epoch_ptr = None
    if mac_cache_ready is not None and mac_cache_ready.numel() > 0:
        _req(mac_cache_ready.is_cuda, "mac_cache_ready must be CUDA")
        _req(mac_cache_ready.is_contiguous(), "mac_cache_ready must be contiguous")
        _req(mac_cache_ready.dtype in (torch.bool, torch.uint8),
             "mac_cache_ready must be bool or uint8")
        _req(mac_cache_ready.numel() >= R, "mac_cache_ready is smaller than the ring")
        ready_ptr = mac_cache_ready.data_ptr()
        if (mac_cache_epoch is not None and mac_cache_epoch.numel() > 0
                and mac_request_epoch is not None and mac_request_epoch.numel() > 0):
            _check(mac_cache_epoch, "mac_cache_epoch", _I64, 1)
            _check(mac_request_epoch, "mac_request_epoch", _I64, 1)
            _req(mac_cache_epoch.numel() >= R and mac_request_epoch.numel() >= R,
                 "epoch tensors are smaller than the ring")
            epoch_ptr = mac_cache_epoch.data_ptr()
            req_epoch_ptr = mac_request_epoch.data_ptr()

    a = _abi.MacB200DecodeArgs()
    a.N, a.Hq, a.Hkv, a.D, a.M, a.R = N, Hq, Hkv, D, M, R
    a.req_to_token_rows, a.req_to_token_stride = req_to_token.shape
    a.kv_tokens = k_buffer.shape[0]
    a.ws_batch, a.max_match_tiles = ws_batch, Tm
    a.max_context, a.tile_tokens, a.match_tile_slots = max_context, tile_tokens, match_tile_slots
    a.semantic_pos_ahead = int(semantic_pos_ahead)
    a.front_sink_tokens = int(front_sink_tokens)
    a.gen_min_limit = int(gen_min_limit)
    a.lookback_right = int(lookback_right)
    a.candidate_mode = int(candidate_mode)
    a.threshold, a.sm_scale = float(threshold), float(sm_scale)
    a.debug_enabled, a.bench_mode = int(debug_enabled), int(bench_mode)
    a.bench_hit_rate, a.bench_hit_rate_std = float(bench_hit_rate), float(bench_hit_rate_std)
    a.bench_skip_ratio = float(bench_skip_ratio)
    a.bench_skip_ratio_std = float(bench_skip_ratio_std)
    a.bench_match_lag_mean = float(bench_match_lag_mean)
    a.bench_match_lag_std = float(bench_match_lag_std)
    a.bench_seed = C.c_int32(int(bench_seed) & 0xFFFFFFFF).value
    a.bench_miss_mask = int(bench_miss_mask)
    a.bench_layer_id = C.c_int32(int(bench_layer_id) & 0xFFFFFFFF).value
    # The reference reads these two from the environment on every launch.
    a.mixed_group_fallback = _env_flag("MAC_PERSISTENT_MIXED_GROUP_FALLBACK", 1)
    a.bench_exact_quota = _env_flag("MAC_BENCH_EXACT_QUOTA", 1)
    a.out_cache_loc_is_i64 = 1 if out_cache_loc.dtype == _I64 else 0
    a.phase_cycles_count = phase_cycles.numel()
    a.grid_cap = _env_int("MAC_PERSISTENT_COOP_CTAS", 0)
    a.q_post, a.q_pre = q_post.data_ptr(), q_pre.data_ptr()
    a.k_buffer, a.v_buffer = k_buffer.data_ptr(), v_buffer.data_ptr()
    a.req_to_token, a.req_ids = req_to_token.data_ptr(), req_ids.data_ptr()
    a.past_lens, a.out_cache_loc = past_lens.data_ptr(), out_cache_loc.data_ptr()
    a.query_cache, a.attn_cache = query_cache.data_ptr(), attn_cache.data_ptr()
    a.lse_cache, a.out = lse_cache.data_ptr(), out.data_ptr()
    a.optional_lse = optional_lse.data_ptr() if optional_lse.numel() > 0 else None
    if optional_lse.numel() > 0:
        _req(optional_lse.numel() >= N * Hq, "optional_lse is smaller than [N,Hq]")
    a.match_dist, a.match_pos = match_dist.data_ptr(), match_pos.data_ptr()
    a.match_slot = match_slot.data_ptr()
    a.head_hit, a.head_match_slot = head_hit.data_ptr(), head_match_slot.data_ptr()
    a.head_match_pos, a.head_prefix_end = head_match_pos.data_ptr(), head_prefix_end.data_ptr()
    a.head_rect_start, a.head_new_end = head_rect_start.data_ptr(), head_new_end.data_ptr()
    a.group_rect_begin, a.group_rect_end = group_rect_begin.data_ptr(), group_rect_end.data_ptr()
    a.group_rect_tiles = group_rect_tiles.data_ptr()
    a.group_tail_begin, a.group_tail_end = group_tail_begin.data_ptr(), group_tail_end.data_ptr()
    a.group_tail_tiles, a.group_mode = group_tail_tiles.data_ptr(), group_mode.data_ptr()
    a.task_counts, a.phase_cycles = task_counts.data_ptr(), phase_cycles.data_ptr()
    a.cache_ready, a.cache_epoch, a.request_epoch = ready_ptr, epoch_ptr, req_epoch_ptr

    return a


_DECODE_ARG_COUNT = 68
_TENSOR_ARGS = tuple(range(0, 43)) + (64, 65, 66, 67)
_ARG_CACHE: dict = {}
_ARG_CACHE_MAX = 64
_ARG_CACHE_ON = os.environ.get("MAC_B200_NO_ARG_CACHE", "0") != "1"


def _decode_key(args):
    """Identity of a call for the marshalling cache: address, shape, dtype and
    contiguity of EVERY tensor argument plus all scalars.  A caching allocator
    can hand the same address to a tensor of another shape or dtype, so the
    address alone does not identify a buffer.  A repeat of the same call
    (serving loops and graph warm-ups pass the same buffers every step) reuses
    the checked argument struct instead of re-validating ~50 tensors."""
    ident = tuple(None if t is None else (t.data_ptr(), t.shape, t.dtype, t.is_contiguous())
                  for t in (args[i] for i in _TENSOR_ARGS))
    return (ident, args[43:64], args[0].device)


def _decode_entry(entry_name, args) -> None:
    lib = _abi.load_library()
    key = _decode_key(args) if _ARG_CACHE_ON else None
    a = _ARG_CACHE.get(key) if key is not None else None
    if a is None:
        a = _decode_call(entry_name, *args)
        if key is not None:
            if len(_ARG_CACHE) >= _ARG_CACHE_MAX:
                _ARG_CACHE.clear()
            _ARG_CACHE[key] = a
    else:
        # the reference re-reads these environment knobs on every launch
        a.mixed_group_fallback = _env_flag("MAC_PERSISTENT_MIXED_GROUP_FALLBACK", 1)
        a.bench_exact_quota = _env_flag("MAC_BENCH_EXACT_QUOTA", 1)
        a.grid_cap = _env_int("MAC_PERSISTENT_COOP_CTAS", 0)
    device = args[0].device
    with torch.cuda.device(device):
        _abi.check(getattr(lib, entry_name)(C.byref(a), _stream_ptr(device)))


def mac_persistent_decode_bf16(*args) -> None:
    """One fused MAC decode step; the reference operator's 68 positional arguments
    (13 tensors, 30 workspace tensors, 21 scalars, ``query_post_cache`` and the
    three readiness-gate tensors; see ``_decode_call`` for the names and
    ``include/mac_b200.h`` for the meaning).  Returns ``None``."""
    if len(args) != _DECODE_ARG_COUNT:
        raise TypeError(f"mac_persistent_decode_bf16() takes {_DECODE_ARG_COUNT} positional "
                        f"arguments ({len(args)} given)")
    _decode_entry("mac_b200_persistent_decode_bf16", args)


def mac_persistent_decode_bf16_lean(q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids,
                                    past_lens, out_cache_loc, query_cache, attn_cache, lse_cache,
                                    out, optional_lse, decisions, *scalars_and_gate) -> None:
    """The decode step without the reference's scheduler scratch.

    The reference operator wants 30 workspace tensors, 4-9 GB of them task lists
    and partial buffers of its own scheduler (``fi_hooks.py:1594-1649`` in the
    reference project) that this kernel never touches.  This entry takes the 13
    data tensors, ``decisions`` = the 18 observable workspace tensors from
    :func:`mac_attention_b200.workspace.make_decision_workspace` (match arrays,
    head/group decision arrays, ``task_counts``, ``phase_cycles``), then the same
    21 scalars, ``query_post_cache`` and the three readiness-gate tensors as the
    full operator.  Same kernel, same results."""
    if len(decisions) != 18:
        raise TypeError("decisions must hold the 18 tensors of make_decision_workspace()")
    if len(scalars_and_gate) != 25:
        raise TypeError("expected 21 scalars, query_post_cache and 3 readiness-gate tensors")
    args = (q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids, past_lens, out_cache_loc,
            query_cache, attn_cache, lse_cache, out, optional_lse,
            *decisions[:16], None, None, None, None, None, None, decisions[16],
            None, None, None, None, None, None, decisions[17], *scalars_and_gate)
    _decode_entry("mac_b200_persistent_decode_bf16", args)


def mac_persistent_decode_bf16_noalloc(*args) -> None:
    """The decode step through ``mac_b200_persistent_decode_bf16_noalloc``: same 68
    arguments and results, scratch in the library's fixed 8 MiB block instead of
    an allocated arena.  For hosts that may not allocate device memory (a
    serving process whose pool owns all of HBM, a sandboxed plugin); raises
    ``RuntimeError`` when the step does not fit the block.  Make the first call
    on a device before any stream capture; overlapping calls on one GPU race."""
    if len(args) != _DECODE_ARG_COUNT:
        raise TypeError(f"mac_persistent_decode_bf16_noalloc() takes {_DECODE_ARG_COUNT} "
                        f"positional arguments ({len(args)} given)")
    _decode_entry("mac_b200_persistent_decode_bf16_noalloc", args)


def mac_prefill_update_cache(
    q_cache, attn_cache, lse_cache, request_length, req_ids, src_q, src_attn, src_lse,
    offsets, lens, capacity, num_heads, head_dim, q_post_cache,
) -> None:
    """Copy the last ``min(len, M)`` prompt rows of each request into its ring."""
    lib = _abi.load_library()
    capacity, num_heads, head_dim = int(capacity), int(num_heads), int(head_dim)
    if capacity <= 0 or req_ids.shape[0] == 0:
        return
    for name, t, dt in (("q_cache", q_cache, _BF16), ("attn_cache", attn_cache, _BF16),
                        ("lse_cache", lse_cache, _F32), ("request_length", request_length, _I32),
                        ("req_ids", req_ids, _I32), ("lens", lens, _I32),
                        ("offsets", offsets, _I32), ("src_q", src_q, _BF16),
                        ("src_attn", src_attn, _BF16), ("src_lse", src_lse, _F32)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.is_contiguous(), f"{name} must be contiguous")
        _req(t.dtype == dt, f"{name} has wrong dtype")
    R = q_cache.shape[0]
    _req(R > 0, "R must be > 0")
    _req(q_cache.dim() == 4, "q_cache must be [R,M,H,D]")
    _req(q_cache.shape[1] == capacity, "capacity (M) mismatch")
    _req(q_cache.shape[2] == num_heads, "num_heads (H) mismatch")
    _req(q_cache.shape[3] == head_dim, "head_dim (D) mismatch")
    _req(attn_cache.shape == q_cache.shape, "attn_cache must match q_cache")
    _req(tuple(lse_cache.shape) == (R, capacity, num_heads), "lse_cache shape mismatch")
    _req(src_q.dim() == 3 and src_q.shape[1] == num_heads and src_q.shape[2] == head_dim,
         "src_q must be [sumN,H,D]")
    _req(src_attn.shape == src_q.shape, "src_attn must match src_q")
    _req(src_lse.dim() == 2 and src_lse.shape[1] == num_heads, "src_lse must be [sumN,H]")
    _req(src_lse.shape[0] == src_q.shape[0], "src_lse row count must match src_q")
    B = req_ids.shape[0]
    _req(offsets.shape[0] == B + 1, "offsets must be [B+1]")
    _req(lens.shape[0] == B, "lens must be [B]")
    _req(request_length.shape[0] in (R, B), "request_length must be [R] or [B]")
    post_ptr = None
    if q_post_cache is not None and q_post_cache.numel() > 0:
        _req(q_post_cache.is_cuda, "q_post_cache must be CUDA")
        _req(q_post_cache.is_contiguous(), "q_post_cache must be contiguous")
        _req(q_post_cache.dtype == _BF16, "q_post_cache has wrong dtype")
        _req(q_post_cache.shape == q_cache.shape, "q_post_cache must match q_cache")
        post_ptr = q_post_cache.data_ptr()
    a = _abi.MacB200PrefillArgs()
    a.R, a.M, a.H, a.D, a.B = R, capacity, num_heads, head_dim, B
    a.src_rows = src_q.shape[0]
    a.request_length_by_batch = 1 if request_length.shape[0] == B else 0
    a.q_cache, a.attn_cache, a.lse_cache = (q_cache.data_ptr(), attn_cache.data_ptr(),
                                            lse_cache.data_ptr())
    a.q_post_cache = post_ptr
    a.request_length, a.req_ids = request_length.data_ptr(), req_ids.data_ptr()
    a.src_q, a.src_attn, a.src_lse = src_q.data_ptr(), src_attn.data_ptr(), src_lse.data_ptr()
    a.offsets, a.lens = offsets.data_ptr(), lens.data_ptr()
    with torch.cuda.device(q_cache.device):
        _abi.check(lib.mac_b200_prefill_update_cache(C.byref(a), _stream_ptr(q_cache.device)))


SINK_NONE, SINK_UNMATCHABLE, SINK_EXCLUDE = 0, 1, 2


def mac_prefill_downdate_update_cache(
    q_cache, attn_cache, lse_cache, request_length, req_ids, src_q, full_attn, full_lse,
    band_attn, band_lse, offsets, lens, capacity, num_heads, head_dim, q_post_cache=None, *,
    band_lse_scale=1.0, sink_mode=SINK_NONE, ready=None, cache_epoch=None, request_epoch=None,
    q_post=None, k_buffer=None, v_buffer=None, req_to_token=None, front_sink_tokens=0,
    semantic_pos_ahead=0, sm_scale=None,
) -> None:
    """One-pass prefill ring build: downdate + ring write + ready mark.

    Equivalent, for the ring, to the reference hook's sequence
    (``flashinfer_hooks.py:2459-2492``)::

        band_lse = band_lse * band_lse_scale
        mac_update_then_downdate_bf16_inplace(full_attn, full_lse, band_attn, band_lse)
        [band_lse = -inf                      if sink_mode == SINK_UNMATCHABLE]
        mac_prefill_update_cache(..., src_q, band_attn, band_lse, ...)
        mac_mark_persistent_ready(ready, cache_epoch, request_epoch, req_ids)   # if given

    but only the rows that reach the ring are downdated and ``band_attn`` /
    ``band_lse`` are left untouched.  ``SINK_EXCLUDE`` additionally removes each
    row's attention over the front-sink tokens, computed from ``q_post`` and the
    paged K/V pool, so that prefill rows are matchable under ``front_sink_tokens > 0``.
    """
    lib = _abi.load_library()
    capacity, num_heads, head_dim = int(capacity), int(num_heads), int(head_dim)
    if capacity <= 0 or req_ids.shape[0] == 0:
        return
    for name, t, dt in (("q_cache", q_cache, _BF16), ("attn_cache", attn_cache, _BF16),
                        ("lse_cache", lse_cache, _F32), ("request_length", request_length, _I32),
                        ("req_ids", req_ids, _I32), ("lens", lens, _I32),
                        ("offsets", offsets, _I32), ("src_q", src_q, _BF16),
                        ("full_attn", full_attn, _BF16), ("band_attn", band_attn, _BF16),
                        ("full_lse", full_lse, None), ("band_lse", band_lse, None)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.is_contiguous(), f"{name} must be contiguous")
        if dt is None:
            _req(t.dtype in _LSE_DTYPES, f"{name} must be float32, bfloat16, or float16; got {t.dtype}")
        else:
            _req(t.dtype == dt, f"{name} has wrong dtype")
    R = q_cache.shape[0]
    _req(R > 0, "R must be > 0")
    _req(q_cache.dim() == 4, "q_cache must be [R,M,H,D]")
    _req(q_cache.shape[1] == capacity, "capacity (M) mismatch")
    _req(q_cache.shape[2] == num_heads, "num_heads (H) mismatch")
    _req(q_cache.shape[3] == head_dim, "head_dim (D) mismatch")
    _req(attn_cache.shape == q_cache.shape, "attn_cache must match q_cache")
    _req(tuple(lse_cache.shape) == (R, capacity, num_heads), "lse_cache shape mismatch")
    _req(src_q.dim() == 3 and src_q.shape[1] == num_heads and src_q.shape[2] == head_dim,
         "src_q must be [sumN,H,D]")
    _req(full_attn.shape == src_q.shape, "full_attn must match src_q")
    _req(band_attn.shape == src_q.shape, "band_attn must match src_q")
    for name, t in (("full_lse", full_lse), ("band_lse", band_lse)):
        _req(t.dim() == 2 and tuple(t.shape) == tuple(src_q.shape[:2]), f"{name} must be [sumN,H]")
    B = req_ids.shape[0]
    _req(offsets.shape[0] == B + 1, "offsets must be [B+1]")
    _req(lens.shape[0] == B, "lens must be [B]")
    _req(request_length.shape[0] in (R, B), "request_length must be [R] or [B]")
    sink_mode = int(sink_mode)
    _req(sink_mode in (SINK_NONE, SINK_UNMATCHABLE, SINK_EXCLUDE), "unknown sink_mode")
    a = _abi.MacB200PrefillBuildArgs()
    r = a.ring
    r.R, r.M, r.H, r.D, r.B = R, capacity, num_heads, head_dim, B
    r.src_rows = src_q.shape[0]
    r.request_length_by_batch = 1 if request_length.shape[0] == B else 0
    r.q_cache, r.attn_cache, r.lse_cache = (q_cache.data_ptr(), attn_cache.data_ptr(),
                                            lse_cache.data_ptr())
    r.q_post_cache = None
    if q_post_cache is not None and q_post_cache.numel() > 0:
        _req(q_post_cache.is_cuda and q_post_cache.is_contiguous(), "q_post_cache must be contiguous CUDA")
        _req(q_post_cache.dtype == _BF16, "q_post_cache has wrong dtype")
        _req(q_post_cache.shape == q_cache.shape, "q_post_cache must match q_cache")
        r.q_post_cache = q_post_cache.data_ptr()
    r.request_length, r.req_ids = request_length.data_ptr(), req_ids.data_ptr()
    r.src_q, r.src_attn, r.src_lse = src_q.data_ptr(), full_attn.data_ptr(), full_lse.data_ptr()
    r.offsets, r.lens = offsets.data_ptr(), lens.data_ptr()
    a.band_attn, a.band_lse = band_attn.data_ptr(), band_lse.data_ptr()
    a.full_lse_dtype, a.band_lse_dtype = _LSE_DTYPES[full_lse.dtype], _LSE_DTYPES[band_lse.dtype]
    a.band_lse_scale = float(band_lse_scale)
    a.sink_mode = sink_mode
    if ready is not None or cache_epoch is not None or request_epoch is not None:
        _req(ready is not None and cache_epoch is not None and request_epoch is not None,
             "ready, cache_epoch and request_epoch go together")
        _check_gate(ready, cache_epoch, request_epoch, req_ids)
        _req(ready.shape[0] == R, "ready must be [R]")
        a.ready, a.cache_epoch, a.request_epoch = (ready.data_ptr(), cache_epoch.data_ptr(),
                                                   request_epoch.data_ptr())
    if sink_mode == SINK_EXCLUDE:
        for name, t in (("q_post", q_post), ("k_buffer", k_buffer), ("v_buffer", v_buffer),
                        ("req_to_token", req_to_token)):
            _req(t is not None, f"{name} is required for SINK_EXCLUDE")
            _req(t.is_cuda and t.is_contiguous(), f"{name} must be contiguous CUDA")
        _req(q_post.dtype == _BF16 and q_post.shape == src_q.shape, "q_post must match src_q")
        _req(k_buffer.dtype == _BF16 and v_buffer.dtype == _BF16, "k_buffer / v_buffer must be bfloat16")
        _req(k_buffer.dim() == 3 and k_buffer.shape[2] == head_dim, "k_buffer must be [T,Hkv,D]")
        _req(v_buffer.shape == k_buffer.shape, "v_buffer must match k_buffer")
        _req(num_heads % k_buffer.shape[1] == 0, "num_heads must be divisible by Hkv")
        _req(req_to_token.dtype == _I32 and req_to_token.dim() == 2, "req_to_token must be int32 [rows,cols]")
        _req(int(front_sink_tokens) >= 0 and int(semantic_pos_ahead) >= 0, "negative F or S")
        a.Hkv = k_buffer.shape[1]
        a.front_sink_tokens, a.semantic_pos_ahead = int(front_sink_tokens), int(semantic_pos_ahead)
        a.req_to_token_rows, a.req_to_token_stride = req_to_token.shape
        a.sm_scale = float(head_dim ** -0.5 if sm_scale is None else sm_scale)
        a.kv_tokens = k_buffer.shape[0]
        a.q_post, a.k_buffer, a.v_buffer = q_post.data_ptr(), k_buffer.data_ptr(), v_buffer.data_ptr()
        a.req_to_token = req_to_token.data_ptr()
    with torch.cuda.device(q_cache.device):
        _abi.check(lib.mac_b200_prefill_downdate_update_cache(C.byref(a), _stream_ptr(q_cache.device)))


def _check_gate(ready, cache_epoch, request_epoch, req_ids) -> None:
    for name, t, dt in (("ready", ready, torch.bool), ("cache_epoch", cache_epoch, _I64),
                        ("request_epoch", request_epoch, _I64), ("req_ids", req_ids, _I32)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.is_contiguous(), f"{name} must be contiguous")
        _req(t.dtype == dt, f"{name} has wrong dtype")
    _req(cache_epoch.shape[0] == ready.shape[0], "cache_epoch must match ready")
    _req(request_epoch.shape[0] == ready.shape[0], "request_epoch must match ready")


def mac_mark_persistent_ready(ready, cache_epoch, request_epoch, req_ids) -> None:
    if req_ids.shape[0] == 0:
        return
    lib = _abi.load_library()
    _check_gate(ready, cache_epoch, request_epoch, req_ids)
    with torch.cuda.device(ready.device):
        _abi.check(lib.mac_b200_mark_persistent_ready(
            ready.data_ptr(), cache_epoch.data_ptr(), request_epoch.data_ptr(),
            req_ids.data_ptr(), req_ids.shape[0], ready.shape[0], _stream_ptr(ready.device)))


def mac_invalidate_persistent_ready(ready, cache_epoch, request_epoch, req_ids) -> None:
    if req_ids.shape[0] == 0:
        return
    lib = _abi.load_library()
    _check_gate(ready, cache_epoch, request_epoch, req_ids)
    with torch.cuda.device(ready.device):
        _abi.check(lib.mac_b200_invalidate_persistent_ready(
            ready.data_ptr(), cache_epoch.data_ptr(), request_epoch.data_ptr(),
            req_ids.data_ptr(), req_ids.shape[0], ready.shape[0], _stream_ptr(ready.device)))


def mac_update_request_state(req_len, match_req_len, cache_lens, req_ids, seq_lens,
                             cur_lens) -> None:
    if req_ids.shape[0] == 0:
        return
    lib = _abi.load_library()
    for name, t in (("req_len", req_len), ("match_req_len", match_req_len),
                    ("cache_lens", cache_lens), ("req_ids", req_ids),
                    ("seq_lens", seq_lens), ("cur_lens", cur_lens)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.is_contiguous(), f"{name} must be contiguous")
        _req(t.dtype == _I32, f"{name} has wrong dtype")
    B = req_ids.shape[0]
    _req(match_req_len.shape[0] == req_len.shape[0], "match_req_len must match req_len")
    _req(seq_lens.shape[0] >= B, "seq_lens is shorter than req_ids")
    _req(cur_lens.shape[0] >= B, "cur_lens is shorter than req_ids")
    _req(cache_lens.shape[0] >= B, "cache_lens is shorter than req_ids")
    with torch.cuda.device(req_len.device):
        _abi.check(lib.mac_b200_update_request_state(
            req_len.data_ptr(), match_req_len.data_ptr(), cache_lens.data_ptr(),
            req_ids.data_ptr(), seq_lens.data_ptr(), cur_lens.data_ptr(), B, req_len.shape[0],
            _stream_ptr(req_len.device)))


def mac_decode_rope_preserve_q_bf16(q, k, v, q_pre, k_buffer, v_buffer, cos_sin_cache, positions,
                                    cache_locs, head_dim, is_neox) -> None:
    """Decode-time fused step before attention: ``q_pre <- q``, RoPE on ``q`` and ``k`` in
    place, rotated ``k`` and ``v`` written to the KV pool at ``cache_locs``.  Arguments and
    checks of the reference operator (``csrc/mac_decode_rope_preserve.cu:174-269``)."""
    lib = _abi.load_library()
    for name, t in (("q", q), ("k", k), ("v", v)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.dtype == _BF16, f"{name} has wrong dtype")
        _req(t.dim() == 2, f"{name} must have rank 2")
        _req(t.stride(1) == 1, f"{name} must have contiguous last dimension")
    for name, t in (("q_pre", q_pre), ("k_buffer", k_buffer), ("v_buffer", v_buffer)):
        _req(t.is_cuda, f"{name} must be CUDA")
        _req(t.dtype == _BF16, f"{name} has wrong dtype")
        _req(t.dim() == 3, f"{name} must have rank 3")
        _req(t.is_contiguous(), f"{name} must be contiguous")
    _req(cos_sin_cache.is_cuda, "cos_sin_cache must be CUDA")
    _req(cos_sin_cache.dtype == _F32, "cos_sin_cache has wrong dtype")
    _req(cos_sin_cache.dim() == 2, "cos_sin_cache must have rank 2")
    _req(cos_sin_cache.stride(1) == 1, "cos_sin_cache must have contiguous last dimension")
    _req(positions.is_cuda and cache_locs.is_cuda, "positions/cache_locs must be CUDA")
    _req(positions.dim() == 1, "positions must have rank 1")
    _req(cache_locs.dim() == 1, "cache_locs must have rank 1")
    _req(positions.dtype in (_I32, _I64), "positions must be int32 or int64")
    _req(cache_locs.dtype in (_I32, _I64), "cache_locs must be int32 or int64")
    _req(positions.is_contiguous() and cache_locs.is_contiguous(),
         "positions/cache_locs must be contiguous")
    head_dim = int(head_dim)
    N = q.shape[0]
    _req(k.shape[0] == N and v.shape[0] == N, "q/k/v batch mismatch")
    _req(positions.shape[0] >= N and cache_locs.shape[0] >= N, "metadata batch too small")
    _req(head_dim > 0 and q.shape[1] % head_dim == 0 and k.shape[1] % head_dim == 0,
         "invalid head_dim")
    Hq, Hkv = q.shape[1] // head_dim, k.shape[1] // head_dim
    _req(v.shape[1] == Hkv * head_dim, "v shape mismatch")
    _req(q_pre.shape[0] >= N and q_pre.shape[1] == Hq and q_pre.shape[2] == head_dim,
         "q_pre shape mismatch")
    _req(k_buffer.shape[1] == Hkv and k_buffer.shape[2] == head_dim, "k_buffer shape mismatch")
    _req(v_buffer.shape == k_buffer.shape, "v_buffer shape mismatch")
    rotary_dim = cos_sin_cache.shape[1]
    _req(0 < rotary_dim <= head_dim and rotary_dim % 2 == 0, "invalid rotary_dim")
    a = _abi.MacB200RopeArgs()
    a.N, a.Hq, a.Hkv, a.head_dim, a.rotary_dim = N, Hq, Hkv, head_dim, rotary_dim
    a.is_neox = 1 if is_neox else 0
    a.positions_i64 = 1 if positions.dtype == _I64 else 0
    a.cache_locs_i64 = 1 if cache_locs.dtype == _I64 else 0
    a.q_stride0, a.k_stride0, a.v_stride0 = q.stride(0), k.stride(0), v.stride(0)
    a.cos_sin_stride0 = cos_sin_cache.stride(0)
    a.kv_pool_tokens = k_buffer.shape[0]
    a.q, a.k, a.v, a.q_pre = q.data_ptr(), k.data_ptr(), v.data_ptr(), q_pre.data_ptr()
    a.k_buffer, a.v_buffer = k_buffer.data_ptr(), v_buffer.data_ptr()
    a.cos_sin_cache = cos_sin_cache.data_ptr()
    a.positions, a.cache_locs = positions.data_ptr(), cache_locs.data_ptr()
    with torch.cuda.device(q.device):
        _abi.check(lib.mac_b200_decode_rope_preserve_q_bf16(C.byref(a), _stream_ptr(q.device)))


_LSE_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def mac_update_then_downdate_bf16_inplace(out1, lse1, out2, lse2) -> None:
    """``(out2, lse2) <- (out1, lse1) minus (out2, lse2)`` per (token, head) row, in place
    (reference operator ``csrc/mac_merge_downdate_cache.cu:320-401``)."""
    lib = _abi.load_library()
    _req(out1.is_cuda and out2.is_cuda, "out tensors must be CUDA")
    _req(lse1.is_cuda and lse2.is_cuda, "lse tensors must be CUDA")
    _req(out1.dtype == _BF16 and out2.dtype == _BF16, "out tensors must be bfloat16")
    _req(out1.dim() == 3, "out1 must be [N,H,D]")
    _req(out2.shape == out1.shape, "out shapes must match [N,H,D]")
    _req(lse1.dim() == 2, "lse1 must be [N,H]")
    _req(lse2.shape == lse1.shape, "lse shapes must match [N,H]")
    _req(tuple(lse1.shape) == tuple(out1.shape[:2]), "lse shapes must match [N,H]")
    _req(out1.is_contiguous() and out2.is_contiguous(), "out tensors must be contiguous")
    _req(lse1.is_contiguous() and lse2.is_contiguous(), "lse tensors must be contiguous")
    _req(out1.device == out2.device == lse1.device == lse2.device,
         "tensors must be on the same device")
    for name, t in (("lse1", lse1), ("lse2", lse2)):
        _req(t.dtype in _LSE_DTYPES, f"{name} must be float32, bfloat16, or float16; got {t.dtype}")
    rows = out1.shape[0] * out1.shape[1]
    with torch.cuda.device(out1.device):
        _abi.check(lib.mac_b200_update_then_downdate_bf16_inplace(
            out1.data_ptr(), lse1.data_ptr(), _LSE_DTYPES[lse1.dtype], out2.data_ptr(),
            lse2.data_ptr(), _LSE_DTYPES[lse2.dtype], rows, out1.shape[2],
            _stream_ptr(out1.device)))


def query_status(device=None) -> int:
    """Sticky device status word (synchronises the current stream); 0 = healthy."""
    lib = _abi.load_library()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    v = C.c_uint32(0)
    with torch.cuda.device(dev):
        _abi.check(lib.mac_b200_query_status(C.byref(v), _stream_ptr(dev)))
    return int(v.value)


def selftest_bounded_wait(device=None):
    """Runs the library's bounded-wait self-test; returns ``(status_word, ctas_that_gave_up)``."""
    lib = _abi.load_library()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status, gave_up = C.c_uint32(0), C.c_int32(0)
    with torch.cuda.device(dev):
        _abi.check(lib.mac_b200_selftest_bounded_wait(C.byref(status), C.byref(gave_up),
                                                      _stream_ptr(dev)))
    return int(status.value), int(gave_up.value)


def launch_info(device=None) -> dict:
    lib = _abi.load_library()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    info = _abi.MacB200LaunchInfo()
    with torch.cuda.device(dev):
        _abi.check(lib.mac_b200_launch_info(C.byref(info)))
    return {name: getattr(info, name) for name, _ in info._fields_}
