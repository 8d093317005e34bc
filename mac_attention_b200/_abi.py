"""ctypes view of ``include/mac_b200.h`` and the library loader."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent

i32, i64, f32 = C.c_int32, C.c_int64, C.c_float
ptr = C.c_void_p


class MacB200DecodeArgs(C.Structure):
    _fields_ = [
        ("N", i32), ("Hq", i32), ("Hkv", i32), ("D", i32), ("M", i32), ("R", i32),
        ("req_to_token_rows", i32), ("req_to_token_stride", i32),
        ("kv_tokens", i64),
        ("ws_batch", i32), ("max_match_tiles", i32),
        ("max_context", i32), ("tile_tokens", i32), ("match_tile_slots", i32),
        ("semantic_pos_ahead", i32), ("front_sink_tokens", i32), ("gen_min_limit", i32),
        ("lookback_right", i32), ("candidate_mode", i32),
        ("threshold", f32), ("sm_scale", f32),
        ("debug_enabled", i32), ("bench_mode", i32),
        ("bench_hit_rate", f32), ("bench_hit_rate_std", f32),
        ("bench_skip_ratio", f32), ("bench_skip_ratio_std", f32),
        ("bench_match_lag_mean", f32), ("bench_match_lag_std", f32),
        ("bench_seed", i32), ("bench_miss_mask", i32), ("bench_layer_id", i32),
        ("mixed_group_fallback", i32), ("bench_exact_quota", i32),
        ("out_cache_loc_is_i64", i32), ("phase_cycles_count", i32), ("grid_cap", i32),
        ("bench_long_band", i32),
        ("q_post", ptr), ("q_pre", ptr), ("k_buffer", ptr), ("v_buffer", ptr),
        ("req_to_token", ptr), ("req_ids", ptr), ("past_lens", ptr), ("out_cache_loc", ptr),
        ("query_cache", ptr), ("attn_cache", ptr), ("lse_cache", ptr),
        ("out", ptr), ("optional_lse", ptr),
        ("match_dist", ptr), ("match_pos", ptr), ("match_slot", ptr),
        ("head_hit", ptr), ("head_match_slot", ptr), ("head_match_pos", ptr),
        ("head_prefix_end", ptr), ("head_rect_start", ptr), ("head_new_end", ptr),
        ("group_rect_begin", ptr), ("group_rect_end", ptr), ("group_rect_tiles", ptr),
        ("group_tail_begin", ptr), ("group_tail_end", ptr), ("group_tail_tiles", ptr),
        ("group_mode", ptr), ("task_counts", ptr), ("phase_cycles", ptr),
        ("cache_ready", ptr), ("cache_epoch", ptr), ("request_epoch", ptr),
    ]


class MacB200PrefillArgs(C.Structure):
    _fields_ = [
        ("R", i32), ("M", i32), ("H", i32), ("D", i32), ("B", i32), ("src_rows", i32),
        ("request_length_by_batch", i32),
        ("q_cache", ptr), ("attn_cache", ptr), ("lse_cache", ptr), ("q_post_cache", ptr),
        ("request_length", ptr), ("req_ids", ptr),
        ("src_q", ptr), ("src_attn", ptr), ("src_lse", ptr),
        ("offsets", ptr), ("lens", ptr),
    ]


class MacB200PrefillBuildArgs(C.Structure):
    _fields_ = [
        ("ring", MacB200PrefillArgs),
        ("band_attn", ptr), ("band_lse", ptr),
        ("full_lse_dtype", i32), ("band_lse_dtype", i32), ("band_lse_scale", C.c_float),
        ("sink_mode", i32),
        ("ready", ptr), ("cache_epoch", ptr), ("request_epoch", ptr),
        ("Hkv", i32), ("front_sink_tokens", i32), ("semantic_pos_ahead", i32),
        ("req_to_token_rows", i32), ("req_to_token_stride", i32), ("sm_scale", C.c_float),
        ("kv_tokens", i64),
        ("q_post", ptr), ("k_buffer", ptr), ("v_buffer", ptr), ("req_to_token", ptr),
    ]


class MacB200RopeArgs(C.Structure):
    _fields_ = [
        ("N", i64), ("Hq", i32), ("Hkv", i32), ("head_dim", i32), ("rotary_dim", i32),
        ("is_neox", i32), ("positions_i64", i32), ("cache_locs_i64", i32), ("reserved", i32),
        ("q_stride0", i64), ("k_stride0", i64), ("v_stride0", i64), ("cos_sin_stride0", i64),
        ("kv_pool_tokens", i64),
        ("q", ptr), ("k", ptr), ("v", ptr), ("q_pre", ptr), ("k_buffer", ptr), ("v_buffer", ptr),
        ("cos_sin_cache", ptr), ("positions", ptr), ("cache_locs", ptr),
    ]


class MacB200LaunchInfo(C.Structure):
    _fields_ = [
        ("sm_count", i32), ("ctas_per_sm", i32), ("block_threads", i32),
        ("dynamic_smem_bytes", i32), ("regs_per_thread", i32), ("last_grid", i32),
        ("arena_bytes", i64), ("kernel_launches", i64),
    ]


# Every symbol include/mac_b200.h declares, with its ctypes prototype.
PROTOTYPES = {
    "mac_b200_persistent_decode_bf16": (C.c_int, [C.POINTER(MacB200DecodeArgs), ptr]),
    "mac_b200_persistent_decode_bf16_noalloc": (C.c_int, [C.POINTER(MacB200DecodeArgs), ptr]),
    "mac_b200_prefill_update_cache": (C.c_int, [C.POINTER(MacB200PrefillArgs), ptr]),
    "mac_b200_prefill_downdate_update_cache": (C.c_int, [C.POINTER(MacB200PrefillBuildArgs), ptr]),
    "mac_b200_mark_persistent_ready": (C.c_int, [ptr, ptr, ptr, ptr, i32, i32, ptr]),
    "mac_b200_invalidate_persistent_ready": (C.c_int, [ptr, ptr, ptr, ptr, i32, i32, ptr]),
    "mac_b200_update_request_state": (C.c_int, [ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, ptr]),
    "mac_b200_decode_rope_preserve_q_bf16": (C.c_int, [C.POINTER(MacB200RopeArgs), ptr]),
    "mac_b200_update_then_downdate_bf16_inplace": (C.c_int, [ptr, ptr, i32, ptr, ptr, i32, i64, i32, ptr]),
    "mac_b200_last_error": (C.c_char_p, []),
    "mac_b200_abi_version": (C.c_int, []),
    "mac_b200_query_status": (C.c_int, [C.POINTER(C.c_uint32), ptr]),
    "mac_b200_launch_info": (C.c_int, [C.POINTER(MacB200LaunchInfo)]),
    "mac_b200_selftest_bounded_wait": (C.c_int, [C.POINTER(C.c_uint32), C.POINTER(C.c_int32), ptr]),
}

ABI_VERSION = 2
_lib = None


def library_path() -> Path:
    return Path(os.environ.get("MAC_B200_LIB", PKG / "libmac_b200.so"))


def load_library() -> C.CDLL:
    """dlopen the CUDA library; build it in-tree when a compiler is here.

    Raises if the library cannot be found or built: there is no other path.
    """
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if "MAC_B200_LIB" not in os.environ:
        from . import build as _build

        try:
            if _build.is_stale():
                _build.build()
        except Exception as exc:  # noqa: BLE001
            if not path.exists():
                raise RuntimeError(
                    f"libmac_b200.so is missing and could not be built: {exc}"
                ) from exc
    if not path.exists():
        raise RuntimeError(f"CUDA library not found: {path}")
    lib = C.CDLL(str(path))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    got = lib.mac_b200_abi_version()
    if got != ABI_VERSION:
        raise RuntimeError(f"libmac_b200.so has ABI version {got}, expected {ABI_VERSION}")
    _lib = lib
    return lib


def check(code: int) -> None:
    """Turn a C-ABI status into the RuntimeError the reference's TORCH_CHECK raises."""
    if code != 0:
        msg = load_library().mac_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"mac_b200: {msg} (code {code})")
