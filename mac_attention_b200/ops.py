"""Operators with the reference extension modules' names and positional signatures.

``mac_persistent_decode_bf16`` takes the 68 positional arguments of the
reference operator (``csrc/mac_decode_persistent.cu:4962-5030`` in the reference
project), ``mac_prefill_update_cache`` and the three gate/state operators take
those of ``csrc/mac_prefill_update_cache.cu:324-337, 374-495``.  Each one checks
what the reference launcher checks (same messages, ``RuntimeError``), fills the
plain-C argument struct and calls the C ABI on torch's current stream.  The
decode operators -- the per-step hot call -- do that in a compiled
torch-extension shim (``csrc/mac_b200_torch.cpp``), the others through ctypes.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _abi

_BF16, _F32, _I32, _I64 = torch.bfloat16, torch.float32, torch.int32, torch.int64


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_DECODE_ARG_COUNT = 68
_shim = None


def _load_shim():
    """The torch-extension shim of the decode operator (``csrc/mac_b200_torch.cpp``): it
    takes the tensors, runs the reference launcher's checks in C++ and calls the C ABI on
    torch's current stream.  Built in-tree next to ``libmac_b200.so``; there is no other
    path to the decode kernel from Python."""
    global _shim
    if _shim is None:
        import importlib.util

        _abi.load_library()
        from . import build as _build

        try:
            if _build.shim_is_stale():
                _build.build_shim()
        except Exception as exc:  # noqa: BLE001
            if not _build.SHIM.exists():
                raise RuntimeError(f"mac_b200_torch.so is missing and could not be built: {exc}") from exc
        spec = importlib.util.spec_from_file_location("mac_b200_torch", _build.SHIM)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _shim = mod
    return _shim


def _raise_on_failure(rc: int) -> None:
    """0 = launched.  A failed check of the shim carries its own text (the message the
    reference's TORCH_CHECK would raise); anything else is a C-ABI status code."""
    if rc == 0:
        return
    if rc == _shim.CHECK_FAILED:
        raise RuntimeError(_shim.last_error())
    _abi.check(rc)


def mac_persistent_decode_bf16(*args) -> None:
    """One fused MAC decode step; the reference operator's 68 positional arguments
    (``csrc/mac_decode_persistent.cu:4962-5030`` in the reference project): 13 tensors,
    30 workspace tensors, 21 scalars, ``query_post_cache`` and the three readiness-gate
    tensors; ``include/mac_b200.h`` has their meaning.  Checks are the reference
    launcher's, with its messages, raised as ``RuntimeError`` before any launch.
    Returns ``None``."""
    if len(args) != _DECODE_ARG_COUNT:
        raise TypeError(f"mac_persistent_decode_bf16() takes {_DECODE_ARG_COUNT} positional "
                        f"arguments ({len(args)} given)")
    _raise_on_failure(_load_shim().decode(0, *args))


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
    _raise_on_failure(_load_shim().decode(
        0, q_post, q_pre, k_buffer, v_buffer, req_to_token, req_ids, past_lens, out_cache_loc,
        query_cache, attn_cache, lse_cache, out, optional_lse,
        *decisions[:16], None, None, None, None, None, None, decisions[16],
        None, None, None, None, None, None, decisions[17], *scalars_and_gate))


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
    _raise_on_failure(_load_shim().decode(1, *args))


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
