"""ctypes binding of libb200kv.so (the C ABI declared in include/b200kv.h).

The library is the product; this module only loads it.  There is no fallback:
if the shared object is missing or a symbol is absent, importing fails.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# B200KV_LIBRARY points the binding at another build of the same library (A/B measurements).
LIB_PATH = Path(os.environ.get("B200KV_LIBRARY") or Path(__file__).resolve().parent / "lib" / "libb200kv.so")


class View(C.Structure):
    """b200kv_view (include/b200kv.h); mirrors MIInfer's AttentionKvCacheView,
    include/miinfer/prefill_v2/kv_cache.hpp:24-46."""

    _fields_ = [
        ("key_f16", C.c_void_p), ("value_f16", C.c_void_p),
        ("key_q8", C.c_void_p), ("key_scales", C.c_void_p),
        ("value_q8", C.c_void_p), ("value_scales", C.c_void_p),
        ("capacity", C.c_uint64), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("qblock", C.c_uint32), ("quant_mode", C.c_uint32),
    ]


u32, u64, sz, vp, fl, i32 = C.c_uint32, C.c_uint64, C.c_size_t, C.c_void_p, C.c_float, C.c_int
VP = C.POINTER(View)


class PoolCounters(C.Structure):
    """b200kv_pool_counters."""
    _fields_ = [("entries", u32), ("bytes", u64), ("hits", u64), ("misses", u64), ("captures", u64), ("evictions", u64), ("skipped", u64)]


class ReuseOptions(C.Structure):
    """b200kv_reuse_options: the prefix-reuse fields of MIInfer's GenerateOptions (include/miinfer/prefill_v2/model.hpp:27-44)."""
    _fields_ = [("enable_prefix_reuse", i32), ("cache_prefix_after", i32), ("cache_prefix_len", u32), ("persistent_session_dir", C.c_char_p)]


class ReuseStats(C.Structure):
    """b200kv_reuse_stats: the reuse telemetry of GenerateStats (model.hpp:61-68)."""
    _fields_ = [("reuse_hit", i32), ("source", i32), ("prefix_tokens_reused", u32), ("suffix_tokens_dispatched", u32),
                ("gqa_kv_reused_tokens", u32), ("restore_ms", C.c_double)]


# name -> (restype, argtypes); one entry per declaration in include/b200kv.h
SIGNATURES = {
    "b200kv_version": (i32, []),
    "b200kv_status_string": (C.c_char_p, [i32]),
    "b200kv_last_cuda_error": (C.c_char_p, []),
    "b200kv_device_check": (i32, [i32]),
    "b200kv_set_launch_overlap": (i32, [u32]),
    "b200kv_set_status_word": (i32, [vp]),
    "b200kv_workspace_reset": (i32, [vp, sz, vp]),
    "b200kv_set_decode_kernel": (i32, [i32]),
    "b200kv_set_timeline_buffer": (i32, [vp, u32]),
    "b200kv_cache_bytes": (sz, [u64, u32, u32, u32, u32]),
    "b200kv_cache_create": (i32, [C.POINTER(vp), u64, u32, u32, u32, u32]),
    "b200kv_cache_destroy": (i32, [vp]),
    "b200kv_cache_reset": (i32, [vp, vp]),
    "b200kv_cache_view": (i32, [vp, VP]),
    "b200kv_append": (i32, [VP, vp, vp, i32, vp, i32, fl, fl, u32, u32, vp, vp, vp]),
    "b200kv_q_split_norm_rope": (i32, [vp, i32, vp, vp, i32, vp, u32, u32, u32, u32, i32, fl, fl, vp, vp, vp]),
    "b200kv_decode_state_advance": (i32, [vp, vp, u32, vp]),
    "b200kv_decode_workspace_bytes": (sz, [u32, u32, u32]),
    "b200kv_decode_attn": (i32, [VP, vp, i32, vp, vp, vp, vp, u32, fl, u32, vp, vp, sz, u32, vp]),
    "b200kv_decode_step": (i32, [VP, vp, vp, i32, vp, i32, fl, fl, vp, i32, vp, vp, vp, vp, u32, fl, u32, vp, vp, sz, u32, vp]),
    "b200kv_decode_static_scratch_bytes": (sz, []),
    "b200kv_decode_attn_static": (i32, [VP, vp, i32, vp, vp, vp, u32, fl, u32, vp, u32, vp]),
    "b200kv_view_table_bytes": (sz, [u32]),
    "b200kv_decode_kernel_kind": (i32, [VP, u32]),
    "b200kv_decode_attn_batched": (i32, [VP, vp, vp, u32, u32, vp, i32, vp, vp, vp, u32, fl, vp, sz, u32, vp]),
    "b200kv_decode_partials": (i32, [VP, vp, i32, u32, fl, u32, u32, vp, vp, vp, vp, sz, u32, vp]),
    "b200kv_exchange_bytes": (sz, [u32, u32, u32]),
    "b200kv_decode_attn_sharded": (i32, [VP, vp, i32, vp, vp, vp, u32, fl, u32, u32, C.POINTER(vp), u32, u32, u32, vp, sz, u32, vp]),
    "b200kv_exchange_create": (i32, [sz, C.POINTER(vp), vp]),
    "b200kv_exchange_open": (i32, [vp, C.POINTER(vp)]),
    "b200kv_exchange_close": (i32, [vp]),
    "b200kv_exchange_destroy": (i32, [vp]),
    "b200kv_merge_partials": (i32, [vp, vp, vp, u32, u32, u32, vp, vp, vp, vp]),
    "b200kv_merge_partials_packed": (i32, [vp, u32, u32, u32, vp, vp, vp, vp]),
    "b200kv_dist_unique_id": (i32, [vp]),
    "b200kv_dist_init": (i32, [C.POINTER(vp), vp, vp, u32, u32, u32, u32]),
    "b200kv_dist_partial": (i32, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
    "b200kv_dist_merge": (i32, [vp, vp, vp, vp, vp]),
    "b200kv_dist_destroy": (i32, [vp]),
    "b200kv_prefill_workspace_bytes": (sz, [u32, u32, u32]),
    "b200kv_prefill_scratch_bytes": (sz, [u64, u32, u32]),
    "b200kv_prefill_split_bytes": (sz, [u32, u32, u32, u32]),
    "b200kv_prefill_attn": (i32, [VP, vp, i32, vp, vp, u32, u32, u32, fl, vp, vp, sz, vp]),
    "b200kv_prefill_prepare": (i32, [VP, u32, u64, vp, sz, vp]),
    "b200kv_prefill_attn_prepared": (i32, [VP, vp, i32, vp, vp, u32, u32, u32, fl, vp, vp, sz, u32, vp]),
    "b200kv_snapshot_bytes": (sz, [VP, u64]),
    "b200kv_snapshot_save": (i32, [VP, u64, vp, vp]),
    "b200kv_snapshot_restore": (i32, [VP, u64, vp, vp]),
    "b200kv_snapshot_clone": (i32, [VP, VP, u64, vp]),
    "b200kv_download_key": (i32, [VP, u64, vp, vp]),
    "b200kv_download_value": (i32, [VP, u64, vp, vp]),
    "b200kv_token_sequence_hash": (u64, [C.POINTER(u32), sz]),
    "b200kv_plan_batched_decode": (i32, [C.POINTER(u32), u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]),
    "b200kv_prefix_match": (i32, [C.c_char_p, C.c_char_p, u32, vp, u32, C.c_char_p, C.c_char_p, vp, u32]),
    "b200kv_session_filename": (i32, [u64, u32, C.c_char_p, sz]),
    "b200kv_session_save": (i32, [C.c_char_p, C.c_char_p, C.c_char_p, vp, u32, VP, u32, vp]),
    "b200kv_session_inspect": (i32, [C.c_char_p, vp, vp, u32]),
    "b200kv_session_load": (i32, [C.c_char_p, C.c_char_p, C.c_char_p, VP, u32, vp, u32, C.POINTER(u32), vp]),
    "b200kv_session_find": (i32, [C.c_char_p, C.c_char_p, C.c_char_p, vp, u32, C.c_char_p, sz, C.POINTER(u32)]),
    "b200kv_session_write": (i32, [C.c_char_p, C.c_char_p, C.c_char_p, vp, u32, vp, u64, u32, u32, u32, u32, u32]),
    "b200kv_pool_create": (i32, [C.POINTER(vp), C.c_char_p, C.c_char_p, u32, u64, u32]),
    "b200kv_pool_destroy": (i32, [vp]),
    "b200kv_pool_capture": (i32, [vp, vp, u32, VP, u32, vp, C.POINTER(i32)]),
    "b200kv_pool_capture_index_only": (i32, [vp, vp, u32, u64, C.POINTER(i32)]),
    "b200kv_pool_lookup": (i32, [vp, C.c_char_p, C.c_char_p, vp, u32, C.POINTER(u32), C.POINTER(u32)]),
    "b200kv_pool_restore": (i32, [vp, vp, u32, VP, u32, vp, C.POINTER(u32)]),
    "b200kv_pool_stats": (i32, [vp, C.POINTER(PoolCounters)]),
    "b200kv_reuse_begin": (i32, [C.POINTER(ReuseOptions), C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, u32, vp, u32, vp, vp, u32, VP, u32, vp,
                                 C.POINTER(ReuseStats)]),
    "b200kv_reuse_commit": (i32, [C.POINTER(ReuseOptions), C.c_char_p, C.c_char_p, vp, vp, u32, VP, u32, vp, C.POINTER(u32), C.POINTER(i32)]),
    "b200kv_session_read": (i32, [C.c_char_p, C.c_char_p, C.c_char_p, u32, u32, u32, u32, u32, vp, u32, C.POINTER(u32), vp, u64]),
}


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m miinfer_b200.build` "
            "(there is no CPU or PyTorch fallback for the KV path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = load()


class B200KvError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib.b200kv_status_string(status).decode()
        detail = lib.b200kv_last_cuda_error().decode() if status == -3 else ""
        super().__init__(f"{where}: {text} ({status}){' — ' + detail if detail else ''}")


def check(status: int, where: str) -> None:
    if status != 0:
        raise B200KvError(status, where)
