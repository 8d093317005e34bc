"""ctypes front end of ``oracle/mac_oracle.c`` (CPU restatement of the MAC decode path).

TEST INFRASTRUCTURE: the checker for the CUDA kernels, never a product path.
Inputs are CPU ``torch`` tensors with the dtypes and shapes of the reference
operators; ring tensors and outputs are updated in place exactly like the
device entry points do.
"""
from __future__ import annotations

import ctypes as C
import math
import subprocess
from dataclasses import dataclass, field
from pathlib import Path

import torch

from mac_attention_b200 import _abi

HERE = Path(__file__).resolve().parent
LIB = HERE / "libmac_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src, hdr = HERE / "mac_oracle.c", HERE.parent / "include" / "mac_b200.h"
    stale = (not LIB.exists()) or LIB.stat().st_mtime < max(src.stat().st_mtime, hdr.stat().st_mtime)
    if force or stale:
        subprocess.run(["make", "-C", str(HERE), "-B", "libmac_oracle.so"], check=True,
                       capture_output=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB))
        _lib.mac_oracle_decode_step.restype = C.c_int
        _lib.mac_oracle_decode_step.argtypes = [C.POINTER(_abi.MacB200DecodeArgs), C.c_void_p, C.c_void_p]
        _lib.mac_oracle_decode_step_rows.restype = C.c_int
        _lib.mac_oracle_decode_step_rows.argtypes = [C.POINTER(_abi.MacB200DecodeArgs), C.c_void_p,
                                                     C.c_void_p, C.c_void_p]
        _lib.mac_oracle_decide.restype = C.c_int
        _lib.mac_oracle_decide.argtypes = [C.POINTER(_abi.MacB200DecodeArgs), C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.mac_oracle_prefill_update_cache.restype = C.c_int
        _lib.mac_oracle_prefill_update_cache.argtypes = [C.POINTER(_abi.MacB200PrefillArgs)]
        for name in ("mac_oracle_mark_persistent_ready", "mac_oracle_invalidate_persistent_ready"):
            fn = getattr(_lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p] * 4 + [C.c_int32, C.c_int32]
        _lib.mac_oracle_update_request_state.restype = C.c_int
        _lib.mac_oracle_update_request_state.argtypes = [C.c_void_p] * 6 + [C.c_int32, C.c_int32]
        _lib.mac_oracle_ring_slot_to_pos.restype = C.c_int
        _lib.mac_oracle_ring_slot_to_pos.argtypes = [C.c_int] * 3
        _lib.mac_oracle_pos_to_ring_slot.restype = C.c_int
        _lib.mac_oracle_pos_to_ring_slot.argtypes = [C.c_int] * 3
        _lib.mac_oracle_ring_distance.restype = C.c_float
        _lib.mac_oracle_ring_distance.argtypes = [C.c_void_p, C.c_void_p]
        _lib.mac_oracle_threshold_distance.restype = C.c_float
        _lib.mac_oracle_threshold_distance.argtypes = [C.c_float, C.c_int]
        _lib.mac_oracle_abi_struct_size.restype = C.c_int
    return _lib


@dataclass
class DecodeConfig:
    """Scalar arguments of the decode operator (reference defaults of its checker)."""
    max_context: int = 131072
    tile_tokens: int = 32
    match_tile_slots: int = 32
    semantic_pos_ahead: int = 256
    front_sink_tokens: int = 0
    gen_min_limit: int = 0
    lookback_right: int = 0
    candidate_mode: int = 0
    threshold: float = 0.45
    sm_scale: float = 1.0 / math.sqrt(128)
    debug_enabled: int = 0
    bench_mode: int = 0
    bench_hit_rate: float = 1.0
    bench_hit_rate_std: float = 0.0
    bench_skip_ratio: float = -1.0
    bench_skip_ratio_std: float = 0.0
    bench_match_lag_mean: float = 64.0
    bench_match_lag_std: float = 0.0
    bench_seed: int = 1
    bench_miss_mask: int = -1
    bench_layer_id: int = 0
    mixed_group_fallback: int = 1
    bench_exact_quota: int = 1
    bench_long_band: int = 0     # benchmark extension of the C ABI (see include/mac_b200.h)

    def scalar_args(self):
        """The 21 scalars in the operator's positional order."""
        return (self.max_context, self.tile_tokens, self.match_tile_slots,
                self.semantic_pos_ahead, self.front_sink_tokens, self.gen_min_limit,
                self.lookback_right, self.candidate_mode, self.threshold, self.sm_scale,
                self.debug_enabled, self.bench_mode, self.bench_hit_rate,
                self.bench_hit_rate_std, self.bench_skip_ratio, self.bench_skip_ratio_std,
                self.bench_match_lag_mean, self.bench_match_lag_std, self.bench_seed,
                self.bench_miss_mask, self.bench_layer_id)


@dataclass
class DecodeResult:
    out: torch.Tensor               # [N,Hq,D] bf16
    out_f32: torch.Tensor           # [N,Hq,D] f32, before rounding
    ring_o_f32: torch.Tensor        # [N,Hq,D] f32 ring state before rounding
    lse: torch.Tensor               # [N,Hq] f32
    head_hit: torch.Tensor
    head_match_slot: torch.Tensor
    head_match_pos: torch.Tensor
    head_prefix_end: torch.Tensor
    head_rect_start: torch.Tensor
    head_new_end: torch.Tensor
    group_rect_begin: torch.Tensor
    group_mode: torch.Tensor
    task_counts: torch.Tensor
    match_dist: torch.Tensor
    match_pos: torch.Tensor
    match_slot: torch.Tensor
    bad_rows: int = 0
    extra: dict = field(default_factory=dict)


def _p(t):
    return None if t is None else t.data_ptr()


def decode_step(q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids, past_lens,
                out_cache_loc, query_cache, attn_cache, lse_cache, cfg: DecodeConfig,
                cache_ready=None, cache_epoch=None, request_epoch=None,
                row_mask=None) -> DecodeResult:
    """One MAC decode step on the CPU; the three ring tensors are updated in place.
    ``row_mask`` (uint8 ``[N]``): rows with 0 are left out of the step while the batch
    size and the other rows' indices stay (the synthetic-decision hash uses both)."""
    for t in (q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids, past_lens, out_cache_loc,
              query_cache, attn_cache, lse_cache):
        assert t.device.type == "cpu" and t.is_contiguous()
    N, Hq, D = q_post.shape
    Hkv = k_buffer.shape[1]
    R, M = query_cache.shape[:2]
    Tm = (M + cfg.match_tile_slots - 1) // cfg.match_tile_slots
    i32 = dict(dtype=torch.int32)
    res = DecodeResult(
        out=torch.zeros(N, Hq, D, dtype=torch.bfloat16),
        out_f32=torch.zeros(N, Hq, D), ring_o_f32=torch.zeros(N, Hq, D),
        lse=torch.zeros(N, Hq),
        head_hit=torch.zeros(N, Hq, **i32), head_match_slot=torch.zeros(N, Hq, **i32),
        head_match_pos=torch.zeros(N, Hq, **i32), head_prefix_end=torch.zeros(N, Hq, **i32),
        head_rect_start=torch.zeros(N, Hq, **i32), head_new_end=torch.zeros(N, Hq, **i32),
        group_rect_begin=torch.zeros(N, Hkv, **i32), group_mode=torch.zeros(N, Hkv, **i32),
        task_counts=torch.zeros(9, **i32),
        match_dist=torch.zeros(N, Hq, Tm), match_pos=torch.zeros(N, Hq, Tm, **i32),
        match_slot=torch.zeros(N, Hq, Tm, **i32),
    )
    a = _abi.MacB200DecodeArgs()
    a.N, a.Hq, a.Hkv, a.D, a.M, a.R = N, Hq, Hkv, D, M, R
    a.req_to_token_rows, a.req_to_token_stride = req_to_token.shape
    a.kv_tokens = k_buffer.shape[0]
    a.ws_batch, a.max_match_tiles = N, Tm
    for name in ("max_context", "tile_tokens", "match_tile_slots", "semantic_pos_ahead",
                 "front_sink_tokens", "gen_min_limit", "lookback_right", "candidate_mode",
                 "threshold", "sm_scale", "debug_enabled", "bench_mode", "bench_hit_rate",
                 "bench_hit_rate_std", "bench_skip_ratio", "bench_skip_ratio_std",
                 "bench_match_lag_mean", "bench_match_lag_std", "bench_seed", "bench_miss_mask",
                 "bench_layer_id", "mixed_group_fallback", "bench_exact_quota", "bench_long_band"):
        setattr(a, name, getattr(cfg, name))
    a.out_cache_loc_is_i64 = 1 if out_cache_loc.dtype == torch.int64 else 0
    a.q_post, a.q_pre, a.k_buffer, a.v_buffer = _p(q_post), _p(q_pre), _p(k_buffer), _p(v_buffer)
    a.req_to_token, a.req_ids, a.past_lens = _p(req_to_token), _p(req_ids), _p(past_lens)
    a.out_cache_loc = _p(out_cache_loc)
    a.query_cache, a.attn_cache, a.lse_cache = _p(query_cache), _p(attn_cache), _p(lse_cache)
    a.out, a.optional_lse = _p(res.out), _p(res.lse)
    a.match_dist, a.match_pos, a.match_slot = _p(res.match_dist), _p(res.match_pos), _p(res.match_slot)
    a.head_hit, a.head_match_slot = _p(res.head_hit), _p(res.head_match_slot)
    a.head_match_pos, a.head_prefix_end = _p(res.head_match_pos), _p(res.head_prefix_end)
    a.head_rect_start, a.head_new_end = _p(res.head_rect_start), _p(res.head_new_end)
    a.group_rect_begin, a.group_mode = _p(res.group_rect_begin), _p(res.group_mode)
    a.task_counts = _p(res.task_counts)
    if cache_ready is not None and cache_ready.numel() > 0:
        ready_u8 = cache_ready.view(torch.uint8) if cache_ready.dtype == torch.bool else cache_ready
        res.extra["ready_keepalive"] = ready_u8
        a.cache_ready = _p(ready_u8)
        if cache_epoch is not None and request_epoch is not None and cache_epoch.numel() > 0:
            a.cache_epoch, a.request_epoch = _p(cache_epoch), _p(request_epoch)
    if row_mask is not None:
        assert row_mask.dtype == torch.uint8 and row_mask.numel() == N and row_mask.is_contiguous()
    res.bad_rows = lib().mac_oracle_decode_step_rows(C.byref(a), _p(res.out_f32),
                                                     _p(res.ring_o_f32), _p(row_mask))
    if res.bad_rows < 0:
        raise RuntimeError("oracle rejected the shapes")
    return res


def decide(q_pre, req_ids, past_lens, query_cache, lse_cache, cfg: DecodeConfig, *, hkv: int,
           req_to_token_shape, cache_ready=None, cache_epoch=None, request_epoch=None):
    """Per-head match decisions only (scan, threshold, synthetic override, front-sink
    demotion; no attention), for shapes whose K/V would not fit the host: returns
    ``(hit, match_slot, match_pos)`` int32 ``[N, Hq]``."""
    for t in (q_pre, req_ids, past_lens, query_cache, lse_cache):
        assert t.device.type == "cpu" and t.is_contiguous()
    N, Hq, D = q_pre.shape
    R, M = query_cache.shape[:2]
    a = _abi.MacB200DecodeArgs()
    a.N, a.Hq, a.Hkv, a.D, a.M, a.R = N, Hq, hkv, D, M, R
    a.req_to_token_rows, a.req_to_token_stride = req_to_token_shape
    a.ws_batch = N
    a.max_match_tiles = (M + cfg.match_tile_slots - 1) // cfg.match_tile_slots
    for name in ("max_context", "tile_tokens", "match_tile_slots", "semantic_pos_ahead",
                 "front_sink_tokens", "gen_min_limit", "lookback_right", "candidate_mode",
                 "threshold", "sm_scale", "debug_enabled", "bench_mode", "bench_hit_rate",
                 "bench_hit_rate_std", "bench_skip_ratio", "bench_skip_ratio_std",
                 "bench_match_lag_mean", "bench_match_lag_std", "bench_seed", "bench_miss_mask",
                 "bench_layer_id", "mixed_group_fallback", "bench_exact_quota", "bench_long_band"):
        setattr(a, name, getattr(cfg, name))
    a.q_pre, a.req_ids, a.past_lens = _p(q_pre), _p(req_ids), _p(past_lens)
    a.query_cache, a.lse_cache = _p(query_cache), _p(lse_cache)
    keep = None
    if cache_ready is not None and cache_ready.numel() > 0:
        keep = cache_ready.view(torch.uint8) if cache_ready.dtype == torch.bool else cache_ready
        a.cache_ready = _p(keep)
        if cache_epoch is not None and request_epoch is not None and cache_epoch.numel() > 0:
            a.cache_epoch, a.request_epoch = _p(cache_epoch), _p(request_epoch)
    hit = torch.zeros(N, Hq, dtype=torch.int32)
    mslot = torch.zeros(N, Hq, dtype=torch.int32)
    mpos = torch.zeros(N, Hq, dtype=torch.int32)
    lib().mac_oracle_decide(C.byref(a), _p(hit), _p(mslot), _p(mpos))
    return hit, mslot, mpos


def prefill_update_cache(q_cache, attn_cache, lse_cache, request_length, req_ids, src_q, src_attn,
                         src_lse, offsets, lens, capacity, num_heads, head_dim,
                         q_post_cache=None) -> None:
    if capacity <= 0 or req_ids.shape[0] == 0:
        return
    a = _abi.MacB200PrefillArgs()
    a.R, a.M, a.H, a.D, a.B = q_cache.shape[0], capacity, num_heads, head_dim, req_ids.shape[0]
    a.src_rows = src_q.shape[0]
    a.request_length_by_batch = 1 if request_length.shape[0] == req_ids.shape[0] else 0
    a.q_cache, a.attn_cache, a.lse_cache = _p(q_cache), _p(attn_cache), _p(lse_cache)
    a.q_post_cache = _p(q_post_cache) if q_post_cache is not None and q_post_cache.numel() else None
    a.request_length, a.req_ids = _p(request_length), _p(req_ids)
    a.src_q, a.src_attn, a.src_lse = _p(src_q), _p(src_attn), _p(src_lse)
    a.offsets, a.lens = _p(offsets), _p(lens)
    lib().mac_oracle_prefill_update_cache(C.byref(a))


def mark_persistent_ready(ready, cache_epoch, request_epoch, req_ids) -> None:
    r = ready.view(torch.uint8) if ready.dtype == torch.bool else ready
    lib().mac_oracle_mark_persistent_ready(_p(r), _p(cache_epoch), _p(request_epoch), _p(req_ids),
                                           req_ids.shape[0], ready.shape[0])


def invalidate_persistent_ready(ready, cache_epoch, request_epoch, req_ids) -> None:
    r = ready.view(torch.uint8) if ready.dtype == torch.bool else ready
    lib().mac_oracle_invalidate_persistent_ready(_p(r), _p(cache_epoch), _p(request_epoch),
                                                 _p(req_ids), req_ids.shape[0], ready.shape[0])


def update_request_state(req_len, match_req_len, cache_lens, req_ids, seq_lens, cur_lens) -> None:
    lib().mac_oracle_update_request_state(_p(req_len), _p(match_req_len), _p(cache_lens),
                                          _p(req_ids), _p(seq_lens), _p(cur_lens),
                                          req_ids.shape[0], req_len.shape[0])


def decode_rope_preserve(q, k, v, q_pre, k_buffer, v_buffer, cos_sin_cache, positions, cache_locs,
                         head_dim, is_neox) -> None:
    """CPU restatement of the decode RoPE + q-preserve + KV write (all tensors updated in place)."""
    a = _abi.MacB200RopeArgs()
    a.N = q.shape[0]
    a.Hq, a.Hkv = q.shape[1] // head_dim, k.shape[1] // head_dim
    a.head_dim, a.rotary_dim = head_dim, cos_sin_cache.shape[1]
    a.is_neox = 1 if is_neox else 0
    a.positions_i64 = 1 if positions.dtype == torch.int64 else 0
    a.cache_locs_i64 = 1 if cache_locs.dtype == torch.int64 else 0
    a.q_stride0, a.k_stride0, a.v_stride0 = q.stride(0), k.stride(0), v.stride(0)
    a.cos_sin_stride0 = cos_sin_cache.stride(0)
    a.kv_pool_tokens = k_buffer.shape[0]
    a.q, a.k, a.v, a.q_pre = _p(q), _p(k), _p(v), _p(q_pre)
    a.k_buffer, a.v_buffer, a.cos_sin_cache = _p(k_buffer), _p(v_buffer), _p(cos_sin_cache)
    a.positions, a.cache_locs = _p(positions), _p(cache_locs)
    fn = lib().mac_oracle_decode_rope_preserve
    fn.restype, fn.argtypes = C.c_int, [C.POINTER(_abi.MacB200RopeArgs)]
    fn(C.byref(a))


def update_then_downdate(out1, lse1, out2, lse2) -> None:
    """CPU restatement of the prefill downdate; float32 LSEs, ``out2``/``lse2`` in place."""
    assert lse1.dtype == torch.float32 and lse2.dtype == torch.float32
    fn = lib().mac_oracle_update_then_downdate
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]
    fn(_p(out1), _p(lse1), _p(out2), _p(lse2), out1.shape[0] * out1.shape[1], out1.shape[2])


def prefill_build(q_cache, attn_cache, lse_cache, request_length, req_ids, src_q, full_attn,
                  full_lse, band_attn, band_lse, offsets, lens, capacity, num_heads, head_dim,
                  q_post_cache=None, *, band_lse_scale=1.0, sink_mode=0, ready=None,
                  cache_epoch=None, request_epoch=None, q_post=None, k_buffer=None, v_buffer=None,
                  req_to_token=None, front_sink_tokens=0, semantic_pos_ahead=0,
                  sm_scale=None) -> None:
    """CPU restatement of the one-pass prefill ring build (float32 LSE inputs)."""
    if capacity <= 0 or req_ids.shape[0] == 0:
        return
    assert full_lse.dtype == torch.float32 and band_lse.dtype == torch.float32
    a = _abi.MacB200PrefillBuildArgs()
    r = a.ring
    r.R, r.M, r.H, r.D, r.B = q_cache.shape[0], capacity, num_heads, head_dim, req_ids.shape[0]
    r.src_rows = src_q.shape[0]
    r.request_length_by_batch = 1 if request_length.shape[0] == req_ids.shape[0] else 0
    r.q_cache, r.attn_cache, r.lse_cache = _p(q_cache), _p(attn_cache), _p(lse_cache)
    r.q_post_cache = _p(q_post_cache) if q_post_cache is not None and q_post_cache.numel() else None
    r.request_length, r.req_ids = _p(request_length), _p(req_ids)
    r.src_q, r.src_attn, r.src_lse = _p(src_q), _p(full_attn), _p(full_lse)
    r.offsets, r.lens = _p(offsets), _p(lens)
    a.band_attn, a.band_lse = _p(band_attn), _p(band_lse)
    a.band_lse_scale, a.sink_mode = float(band_lse_scale), int(sink_mode)
    keep = []
    if ready is not None:
        rd = ready.view(torch.uint8) if ready.dtype == torch.bool else ready
        keep.append(rd)
        a.ready, a.cache_epoch, a.request_epoch = _p(rd), _p(cache_epoch), _p(request_epoch)
    if int(sink_mode) == 2:
        a.Hkv = k_buffer.shape[1]
        a.front_sink_tokens, a.semantic_pos_ahead = int(front_sink_tokens), int(semantic_pos_ahead)
        a.req_to_token_rows, a.req_to_token_stride = req_to_token.shape
        a.sm_scale = float(head_dim ** -0.5 if sm_scale is None else sm_scale)
        a.kv_tokens = k_buffer.shape[0]
        a.q_post, a.k_buffer, a.v_buffer = _p(q_post), _p(k_buffer), _p(v_buffer)
        a.req_to_token = _p(req_to_token)
    fn = lib().mac_oracle_prefill_build
    fn.restype, fn.argtypes = C.c_int, [C.POINTER(_abi.MacB200PrefillBuildArgs)]
    fn(C.byref(a))


def ring_slot_to_pos(past_len, M, slot):
    return lib().mac_oracle_ring_slot_to_pos(past_len, M, slot)


def pos_to_ring_slot(past_len, M, pos):
    return lib().mac_oracle_pos_to_ring_slot(past_len, M, pos)


def threshold_distance(threshold, D=128):
    return lib().mac_oracle_threshold_distance(threshold, D)


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative L2 error, the reference's stated output metric."""
    x, ref = x.double(), ref.double()
    den = ref.norm().item()
    return (x - ref).norm().item() / (den if den > 0 else 1.0)
