"""Python mirror of MIInfer's KV-cache operator interface over the B200 library.

Names and argument meaning follow the reference's C++ interface so call sites
read the same: KvCacheQuantMode / AttentionKvCacheView /
AttentionLayerKvCacheStorage (include/miinfer/prefill_v2/kv_cache.hpp) and the
three launchers of include/miinfer/qwen3_gpu_primitives.hpp:670-739.  Tensors are
torch CUDA tensors used only as device buffers; all arithmetic runs in
libb200kv.so.  Argument errors raise B200KvError (the reference aborts).
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional

import torch

from ._lib import B200KvError, PoolCounters, ReuseOptions, ReuseStats, View, check, lib

__all__ = [
    "KvCacheQuantMode", "RopeMode", "AttentionKvCacheView", "AttentionLayerKvCacheStorage",
    "launch_kv_store_quant", "launch_decode_attention_quant", "launch_decode_attention_batched", "launch_decode_step",
    "launch_decode_partials", "launch_merge_partials", "launch_merge_partials_packed", "packed_partial", "partial_views", "launch_suffix_attention_quant", "prepare_suffix_attention", "plan_batched_decode",
    "Exchange", "launch_decode_attention_sharded", "decode_workspace", "prefill_workspace", "view_table", "make_decode_state", "make_prefill_state",
    "SnapshotPool", "ReusableContext", "DistMerge", "launch_q_split_norm_rope", "launch_decode_state_advance", "q8_1_blocks", "exchange_words", "set_status_word", "workspace_reset", "set_decode_kernel",
    "token_sequence_hash", "save_session", "load_session", "find_matching_session", "decode_kernel_kind", "set_launch_overlap", "B200KvError", "FORCE_GENERIC",
]

FORCE_GENERIC = 0x80000000


class KvCacheQuantMode(enum.IntEnum):
    """kv_cache.hpp:16-21."""
    kFp16Fp16 = 0
    kQ8Fp16 = 1
    kFp16Q8 = 2
    kQ8Q8 = 3


class RopeMode(enum.IntEnum):
    NONE = 0
    NEOX_FULL = 1
    SECTIONED64 = 2


AttentionKvCacheView = View


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    return t.data_ptr()


def _dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise ValueError(f"unsupported dtype {t.dtype}: fp16 or fp32 expected")


def _stream(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


class AttentionLayerKvCacheStorage:
    """Owns one layer's planes (kv_cache.hpp:49-122, src/prefill_v2/kv_cache.cpp).

    The reference fixes kv_heads=4, head_dim=256 and one scale per row; here
    they are constructor arguments and `qblock=32` selects the q8_0 format.
    """

    def __init__(self, capacity: int, quant_mode: KvCacheQuantMode = KvCacheQuantMode.kFp16Fp16, *,
                 kv_heads: int = 4, head_dim: int = 256, qblock: Optional[int] = None,
                 device: Optional[torch.device] = None):
        if capacity <= 0:
            raise RuntimeError("AttentionLayerKvCacheStorage: capacity must be > 0")  # kv_cache.cpp:12-14
        self.capacity, self.kv_heads, self.head_dim = int(capacity), int(kv_heads), int(head_dim)
        self.qblock = int(qblock if qblock is not None else head_dim)
        self.quant_mode = KvCacheQuantMode(quant_mode)
        if self.head_dim % self.qblock:
            raise ValueError("qblock must divide head_dim")
        dev = device or torch.device("cuda", torch.cuda.current_device())
        rows = self.kv_heads * self.capacity
        nblk = self.head_dim // self.qblock
        k_q8 = self.quant_mode in (KvCacheQuantMode.kQ8Fp16, KvCacheQuantMode.kQ8Q8)
        v_q8 = self.quant_mode in (KvCacheQuantMode.kFp16Q8, KvCacheQuantMode.kQ8Q8)
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        shape = (self.kv_heads, self.capacity, self.head_dim)
        sshape = (self.kv_heads, self.capacity, nblk)
        self.key_cache = None if k_q8 else z(shape, torch.float16)
        self.value_cache = None if v_q8 else z(shape, torch.float16)
        self.key_cache_q8 = z(shape, torch.int8) if k_q8 else None
        self.key_scales = z(sshape, torch.float16) if k_q8 else None
        self.value_cache_q8 = z(shape, torch.int8) if v_q8 else None
        self.value_scales = z(sshape, torch.float16) if v_q8 else None
        del rows

    def planes(self):
        return [t for t in (self.key_cache, self.value_cache, self.key_cache_q8, self.key_scales,
                            self.value_cache_q8, self.value_scales) if t is not None]

    def reset(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        with torch.cuda.stream(stream or torch.cuda.current_stream()):
            for t in self.planes():
                t.zero_()

    def view(self) -> View:
        return View(_ptr(self.key_cache), _ptr(self.value_cache), _ptr(self.key_cache_q8), _ptr(self.key_scales),
                    _ptr(self.value_cache_q8), _ptr(self.value_scales), self.capacity, self.kv_heads,
                    self.head_dim, self.qblock, int(self.quant_mode))

    def total_bytes(self) -> int:
        return int(lib.b200kv_cache_bytes(self.capacity, self.kv_heads, self.head_dim, self.qblock, int(self.quant_mode)))

    def raw_tokens_bytes(self, tokens: int) -> int:
        """kv_cache.cpp:214-225."""
        v = self.view()
        return int(lib.b200kv_snapshot_bytes(C.byref(v), tokens))

    def download_raw(self, dst: torch.Tensor, tokens: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        """kv_cache.cpp:227-297.  dst: uint8 tensor (CUDA, or CPU -- pinned for an async copy)."""
        if tokens > self.capacity:
            raise RuntimeError("AttentionLayerKvCacheStorage::download_raw: tokens exceeds capacity")
        if dst.numel() * dst.element_size() < self.raw_tokens_bytes(tokens):
            raise ValueError("snapshot buffer too small")
        v = self.view()
        check(lib.b200kv_snapshot_save(C.byref(v), tokens, dst.data_ptr(), _stream(stream)), "b200kv_snapshot_save")

    def upload_raw(self, src: torch.Tensor, tokens: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        """kv_cache.cpp:299-369."""
        if tokens > self.capacity:
            raise RuntimeError("AttentionLayerKvCacheStorage::upload_raw: tokens exceeds capacity")
        if src.numel() * src.element_size() < self.raw_tokens_bytes(tokens):
            raise ValueError("snapshot buffer too small")
        v = self.view()
        check(lib.b200kv_snapshot_restore(C.byref(v), tokens, src.data_ptr(), _stream(stream)), "b200kv_snapshot_restore")

    def download_key(self, tokens: int):
        """kv_cache.cpp:132-170: the first `tokens` positions of K as a float32 numpy array [kv_head][tokens][head_dim], dequantised."""
        return self._download(tokens, lib.b200kv_download_key)

    def download_value(self, tokens: int):
        """kv_cache.cpp:172-212."""
        return self._download(tokens, lib.b200kv_download_value)

    def _download(self, tokens: int, fn):
        import numpy as np

        if tokens > self.capacity:
            raise RuntimeError("AttentionLayerKvCacheStorage: tokens exceeds capacity")   # kv_cache.cpp:133-135
        out = np.empty((self.kv_heads, tokens, self.head_dim), np.float32)
        v = self.view()
        check(fn(C.byref(v), tokens, out.ctypes.data, _stream(None)), "b200kv_download")
        return out

    def clone_prefix_from(self, other: "AttentionLayerKvCacheStorage", tokens: int,
                          stream: Optional[torch.cuda.Stream] = None) -> None:
        """Device-to-device copy of the first `tokens` positions (tools/miinfer_cli.cpp:1248-1317)."""
        d, s = self.view(), other.view()
        check(lib.b200kv_snapshot_clone(C.byref(d), C.byref(s), tokens, _stream(stream)), "b200kv_snapshot_clone")


def make_decode_state(position: int, device=None) -> torch.Tensor:
    """A DeviceDecodeState (qwen3_gpu_primitives.hpp:30-37) as a 16-word uint32 tensor."""
    t = torch.zeros(16, dtype=torch.int32, device=device or "cuda")
    t[1] = position
    return t


def make_prefill_state(base_position: int, token_count: int, kv_capacity: int = 0, device=None) -> torch.Tensor:
    """A DevicePrefillState (qwen3_gpu_primitives.hpp:39-45)."""
    t = torch.zeros(16, dtype=torch.int32, device=device or "cuda")
    t[0], t[1], t[2], t[3] = base_position, token_count, base_position + token_count, kv_capacity
    return t


def decode_workspace(query_heads: int, head_dim: int, sessions: int = 1, device=None) -> torch.Tensor:
    n = int(lib.b200kv_decode_workspace_bytes(query_heads, head_dim, sessions))
    return torch.zeros(n, dtype=torch.uint8, device=device or "cuda")   # zero-filled once: the tagged partials in its front part must start at zero


def view_table(sessions: int, device=None) -> torch.Tensor:
    """Device scratch for launch_decode_attention_batched (views + TMA descriptors per session)."""
    return torch.zeros(int(lib.b200kv_view_table_bytes(sessions)), dtype=torch.uint8, device=device or "cuda")


def prefill_workspace(rows: int, kv_heads: int, head_dim: int, device=None, *, token_count: int = 0,
                      query_heads: int = 0) -> torch.Tensor:
    """Scratch that lets launch_suffix_attention_quant run the tcgen05 kernel: `rows` = base_position + token_count.
    With token_count and query_heads given it also has room for the partials of a KV-split launch."""
    n = int(lib.b200kv_prefill_scratch_bytes(rows, kv_heads, head_dim))
    if token_count and query_heads:
        n += int(lib.b200kv_prefill_split_bytes(token_count, query_heads, kv_heads, head_dim))
    return torch.zeros(n, dtype=torch.uint8, device=device or "cuda")


def launch_kv_store_quant(view: View, key: torch.Tensor, value: torch.Tensor, k_norm_weight: Optional[torch.Tensor],
                          token_count: int, base_position: int, *, rope_mode: RopeMode = RopeMode.SECTIONED64,
                          theta: float = 1.0e6, epsilon: float = 1.0e-6,
                          prefill_state: Optional[torch.Tensor] = None, decode_state: Optional[torch.Tensor] = None,
                          stream: Optional[torch.cuda.Stream] = None) -> None:
    """launch_qwen35_decoupled_k_norm_rope_kv_store_batch_quant (qwen3_gpu_primitives.hpp:695-716).

    key/value: [token][kv_heads*head_dim] fp16 or fp32; the cache planes and
    quant mode travel in `view`."""
    if key.dtype != value.dtype:
        raise ValueError("key and value must share a dtype")
    check(lib.b200kv_append(C.byref(view), _ptr(key), _ptr(value), _dtype(key), _ptr(k_norm_weight), int(rope_mode),
                            theta, epsilon, token_count, base_position, _ptr(prefill_state), _ptr(decode_state),
                            _stream(stream)), "b200kv_append")


def launch_q_split_norm_rope(qfull: torch.Tensor, q_norm_weight: Optional[torch.Tensor], query: torch.Tensor,
                             gate: Optional[torch.Tensor], token_count: int, base_position: int, *, heads: int, head_dim: int,
                             rope_mode: RopeMode = RopeMode.SECTIONED64, theta: float = 1.0e6, epsilon: float = 1.0e-6,
                             prefill_state: Optional[torch.Tensor] = None, decode_state: Optional[torch.Tensor] = None,
                             stream: Optional[torch.cuda.Stream] = None) -> None:
    """launch_qwen35_decoupled_q_split_norm_rope_batch / launch_qwen35_fused_q_split_norm_rope_dynamic
    (qwen3_gpu_primitives.hpp:869-881, 934-938): qfull [token][heads][q | gate] -> query, gate [token][heads][d]."""
    check(lib.b200kv_q_split_norm_rope(_ptr(qfull), _dtype(qfull), _ptr(q_norm_weight), _ptr(query), _dtype(query), _ptr(gate),
                                       token_count, base_position, heads, head_dim, int(rope_mode), theta, epsilon,
                                       _ptr(prefill_state), _ptr(decode_state), _stream(stream)), "b200kv_q_split_norm_rope")


def launch_decode_state_advance(state: torch.Tensor, token_output: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
    """launch_qwen35_decode_state_advance (qwen3_gpu_primitives.hpp:1248-1250): device-side position/generated advance."""
    check(lib.b200kv_decode_state_advance(_ptr(state), _ptr(token_output), token_output.numel(), _stream(stream)),
          "b200kv_decode_state_advance")


def launch_decode_attention_quant(view: View, q: torch.Tensor, *, query_heads: int, scale: float,
                                  cache_length: int = 0, decode_state: Optional[torch.Tensor] = None,
                                  output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                                  gated_output: Optional[torch.Tensor] = None, gated_output_q8: Optional[torch.Tensor] = None,
                                  workspace: torch.Tensor, num_splits: int = 0,
                                  stream: Optional[torch.cuda.Stream] = None) -> None:
    """launch_qwen35_tiled_online_attention_quant_dynamic (qwen3_gpu_primitives.hpp:719-739).
    gated_output_q8: uint8 tensor of query_heads * head_dim / 32 Q8_1 blocks (36 bytes each), see `q8_1_blocks`."""
    check(lib.b200kv_decode_attn(C.byref(view), _ptr(q), _dtype(q), _ptr(gate), _ptr(output), _ptr(gated_output), _ptr(gated_output_q8),
                                 query_heads, scale, cache_length, _ptr(decode_state),
                                 _ptr(workspace),
                                 workspace.numel(), num_splits, _stream(stream)), "b200kv_decode_attn")


def launch_decode_step(view: View, key: torch.Tensor, value: torch.Tensor, q: torch.Tensor, *, query_heads: int, scale: float,
                       position: int = 0, decode_state: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                       rope_mode: RopeMode = RopeMode.NEOX_FULL, theta: float = 1.0e6, epsilon: float = 1.0e-6,
                       output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                       gated_output: Optional[torch.Tensor] = None, gated_output_q8: Optional[torch.Tensor] = None,
                       workspace: torch.Tensor, num_splits: int = 0,
                       stream: Optional[torch.cuda.Stream] = None) -> None:
    """Append one token and attend in one launch (b200kv_decode_step): the fused form of the store + decode-attention
    call pair of src/prefill_v2/attention_layer.cpp:599-632."""
    if key.dtype != value.dtype:
        raise ValueError("key and value must share a dtype")
    check(lib.b200kv_decode_step(C.byref(view), _ptr(key), _ptr(value), _dtype(key), _ptr(k_norm_weight), int(rope_mode), theta,
                                 epsilon, _ptr(q), _dtype(q), _ptr(gate), _ptr(output), _ptr(gated_output), _ptr(gated_output_q8),
                                 query_heads, scale,
                                 position, _ptr(decode_state), _ptr(workspace),
                                 workspace.numel(), num_splits, _stream(stream)),
          "b200kv_decode_step")


def launch_decode_attention_batched(views, view_table: torch.Tensor, lengths: torch.Tensor, max_length: int,
                                    q: torch.Tensor, *, query_heads: int, scale: float,
                                    output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                                    gated_output: Optional[torch.Tensor] = None, workspace: torch.Tensor,
                                    num_splits: int = 0, stream: Optional[torch.cuda.Stream] = None) -> None:
    """One decode step for many sessions in one launch (b200kv_decode_attn_batched).

    views: sequence of View, or None to reuse the table filled by an earlier call."""
    sessions = int(lengths.numel())
    arr = None
    if views is not None:
        arr = (View * sessions)(*views)
    check(lib.b200kv_decode_attn_batched(arr, _ptr(view_table), _ptr(lengths), sessions, max_length, _ptr(q), _dtype(q),
                                         _ptr(gate), _ptr(output), _ptr(gated_output), query_heads, scale,
                                         _ptr(workspace), workspace.numel(), num_splits, _stream(stream)),
          "b200kv_decode_attn_batched")


def launch_decode_partials(view: View, q: torch.Tensor, *, query_heads: int, scale: float, range_begin: int,
                           range_end: int, part_m: torch.Tensor, part_l: torch.Tensor, part_acc: torch.Tensor,
                           workspace: torch.Tensor, num_splits: int = 0,
                           stream: Optional[torch.cuda.Stream] = None) -> None:
    check(lib.b200kv_decode_partials(C.byref(view), _ptr(q), _dtype(q), query_heads, scale, range_begin, range_end,
                                     _ptr(part_m), _ptr(part_l), _ptr(part_acc), _ptr(workspace), workspace.numel(),
                                     num_splits, _stream(stream)), "b200kv_decode_partials")


class Exchange:
    """The exchange buffers of sequence-sharded decode on one node: this rank's own buffer plus every peer's,
    mapped into this process.  `handles` are the 64-byte handles of all ranks in rank order (this rank's own
    entry comes from `Exchange.create`); see `partition.open_exchange` for the all-gather that collects them."""

    def __init__(self, own_ptr: int, own_handle: bytes, rank: int):
        self.own_ptr, self.own_handle, self.rank = own_ptr, own_handle, rank
        self.ptrs: list[int] = []
        self._table = None

    @staticmethod
    def create(query_heads: int, head_dim: int, world: int, rank: int) -> "Exchange":
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(lib.b200kv_exchange_create(lib.b200kv_exchange_bytes(query_heads, head_dim, world), C.byref(ptr), handle),
              "b200kv_exchange_create")
        return Exchange(ptr.value, handle.raw, rank)

    @staticmethod
    def from_pointers(ptrs: list, rank: int) -> "Exchange":
        """Exchange over buffers the caller already holds device pointers to (all ranks in one process, tests)."""
        ex = Exchange(0, b"", rank)
        ex.ptrs = [int(x) for x in ptrs]
        ex._table = (C.c_void_p * len(ex.ptrs))(*ex.ptrs)
        return ex

    def open_peers(self, handles: list) -> None:
        self.ptrs = []
        for w, h in enumerate(handles):
            if w == self.rank:
                self.ptrs.append(self.own_ptr)
                continue
            peer = C.c_void_p()
            check(lib.b200kv_exchange_open(C.create_string_buffer(bytes(h), 64), C.byref(peer)), "b200kv_exchange_open")
            self.ptrs.append(peer.value)
        self._table = (C.c_void_p * len(self.ptrs))(*self.ptrs)

    @property
    def world(self) -> int:
        return len(self.ptrs)

    def close(self) -> None:
        if self.own_ptr:   # peers were mapped by open_peers
            for w, ptr in enumerate(self.ptrs):
                if w != self.rank:
                    lib.b200kv_exchange_close(ptr)
        self.ptrs = []

    def destroy(self) -> None:
        self.close()
        if self.own_ptr:
            lib.b200kv_exchange_destroy(self.own_ptr)
            self.own_ptr = 0


def launch_decode_attention_sharded(view: View, q: torch.Tensor, exchange: Exchange, *, query_heads: int, scale: float,
                                    range_begin: int, range_end: int, phase: int, workspace: torch.Tensor,
                                    output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                                    gated_output: Optional[torch.Tensor] = None, num_splits: int = 0,
                                    stream: Optional[torch.cuda.Stream] = None) -> None:
    """Sequence-sharded decode with the cross-GPU merge inside the kernel (b200kv_decode_attn_sharded)."""
    check(lib.b200kv_decode_attn_sharded(C.byref(view), _ptr(q), _dtype(q), _ptr(gate), _ptr(output), _ptr(gated_output),
                                         query_heads, scale, range_begin, range_end, exchange._table, exchange.rank,
                                         exchange.world, phase, _ptr(workspace), workspace.numel(), num_splits,
                                         _stream(stream)), "b200kv_decode_attn_sharded")


class DistMerge:
    """b200kv_dist_*: the NCCL form of the cross-GPU merge for a C or C++ host.  `unique_id()` on one rank, passed
    to the others (any transport), then every rank constructs a DistMerge; per layer: launch_decode_partials with
    `self.partial` and `merge(output=...)`."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib.b200kv_dist_unique_id(buf), "b200kv_dist_unique_id")
        return buf.raw

    def __init__(self, unique_id: bytes, rank: int, world: int, query_heads: int, head_dim: int):
        self._h = C.c_void_p()
        check(lib.b200kv_dist_init(C.byref(self._h), None, C.create_string_buffer(unique_id, 128), rank, world, query_heads, head_dim),
              "b200kv_dist_init")
        m, l, a = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(lib.b200kv_dist_partial(self._h, C.byref(m), C.byref(l), C.byref(a)), "b200kv_dist_partial")
        self.partial_ptrs = (m.value, l.value, a.value)
        self.query_heads, self.head_dim = query_heads, head_dim

    def decode_partials(self, view: View, q: torch.Tensor, *, scale: float, range_begin: int, range_end: int, workspace: torch.Tensor,
                        num_splits: int = 0, stream: Optional[torch.cuda.Stream] = None) -> None:
        m, l, a = self.partial_ptrs
        check(lib.b200kv_decode_partials(C.byref(view), _ptr(q), _dtype(q), self.query_heads, scale, range_begin, range_end, m, l, a,
                                         _ptr(workspace), workspace.numel(), num_splits, _stream(stream)), "b200kv_decode_partials")

    def merge(self, *, output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
              gated_output: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> None:
        check(lib.b200kv_dist_merge(self._h, _ptr(gate), _ptr(output), _ptr(gated_output), _stream(stream)), "b200kv_dist_merge")

    def destroy(self) -> None:
        if self._h:
            lib.b200kv_dist_destroy(self._h)
            self._h = C.c_void_p()


def launch_merge_partials(part_m: torch.Tensor, part_l: torch.Tensor, part_acc: torch.Tensor, *, num_parts: int,
                          query_heads: int, head_dim: int, output: Optional[torch.Tensor] = None,
                          gate: Optional[torch.Tensor] = None, gated_output: Optional[torch.Tensor] = None,
                          stream: Optional[torch.cuda.Stream] = None) -> None:
    check(lib.b200kv_merge_partials(_ptr(part_m), _ptr(part_l), _ptr(part_acc), num_parts, query_heads, head_dim,
                                    _ptr(gate), _ptr(output), _ptr(gated_output), _stream(stream)),
          "b200kv_merge_partials")


def packed_partial(query_heads: int, head_dim: int, parts: int = 1, device=None) -> torch.Tensor:
    """[parts][ m[H] | l[H] | acc[H][d] ] fp32: one rank's partial (parts=1) or the all-gathered set."""
    return torch.zeros(parts, query_heads * (head_dim + 2), dtype=torch.float32, device=device or "cuda")


def partial_views(packed_row: torch.Tensor, query_heads: int, head_dim: int):
    """(m, l, acc) views into one packed partial, to pass to launch_decode_partials."""
    m = packed_row[:query_heads]
    l = packed_row[query_heads:2 * query_heads]
    acc = packed_row[2 * query_heads:].view(query_heads, head_dim)
    return m, l, acc


def launch_merge_partials_packed(packed: torch.Tensor, *, num_parts: int, query_heads: int, head_dim: int,
                                 output: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                                 gated_output: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> None:
    check(lib.b200kv_merge_partials_packed(_ptr(packed), num_parts, query_heads, head_dim, _ptr(gate), _ptr(output),
                                           _ptr(gated_output), _stream(stream)), "b200kv_merge_partials_packed")


def launch_suffix_attention_quant(view: View, q: torch.Tensor, gate: Optional[torch.Tensor], gated_output: torch.Tensor,
                                  workspace: Optional[torch.Tensor], token_count: int, base_position: int, *, query_heads: int,
                                  scale: float, prefill_state: Optional[torch.Tensor] = None, prepared_rows: int = 0,
                                  stream: Optional[torch.cuda.Stream] = None) -> None:
    """launch_qwen35_splitk_suffix_attention_quant (qwen3_gpu_primitives.hpp:670-692).  `prepared_rows`: cache positions
    whose fp16 copy `prepare_suffix_attention` has already put into this workspace."""
    check(lib.b200kv_prefill_attn_prepared(C.byref(view), _ptr(q), _dtype(q), _ptr(gate), _ptr(gated_output), token_count,
                                           base_position, query_heads, scale, _ptr(prefill_state), _ptr(workspace),
                                           0 if workspace is None else workspace.numel(), prepared_rows, _stream(stream)),
          "b200kv_prefill_attn_prepared")


def plan_batched_decode(lengths, kv_heads: int, cta_slots: int = 0):
    """b200kv_plan_batched_decode: (num_splits, max_length) to pass to launch_decode_attention_batched for sessions of
    these lengths (host integers).  Host arithmetic only."""
    arr = (C.c_uint32 * max(1, len(lengths)))(*[int(x) for x in lengths])
    splits, bound = C.c_uint32(0), C.c_uint32(0)
    check(lib.b200kv_plan_batched_decode(arr, len(lengths), kv_heads, cta_slots, C.byref(splits), C.byref(bound)),
          "b200kv_plan_batched_decode")
    return int(splits.value), int(bound.value)


def prepare_suffix_attention(view: View, prepared_rows: int, rows: int, workspace: torch.Tensor,
                             stream: Optional[torch.cuda.Stream] = None) -> None:
    """b200kv_prefill_prepare: the tcgen05 suffix kernel's pre-pass over positions [0, prepared_rows), ahead of the
    attention call that sees `rows` positions and is told `prepared_rows` -- on a second stream it runs beside the
    previous layer's attention."""
    check(lib.b200kv_prefill_prepare(C.byref(view), prepared_rows, rows, _ptr(workspace), workspace.numel(), _stream(stream)),
          "b200kv_prefill_prepare")


def q8_1_blocks(query_heads: int, head_dim: int, device=None) -> torch.Tensor:
    """Room for the Q8_1 form of one decode output: query_heads * head_dim / 32 blocks of 36 bytes
    (fp16 d, fp16 s, 32 int8; Q8_1Block, include/miinfer/q4_q8_gemv.hpp:23-27)."""
    return torch.zeros(query_heads * head_dim // 32, 36, dtype=torch.uint8, device=device or "cuda")


def exchange_words(values: torch.Tensor, phase: int) -> torch.Tensor:
    """fp32 values as the 8-byte words of call number `phase` of a sequence-sharded exchange: the value in the low
    half, the call's tag (phase + 1) in the high half.  Tests use it to play a peer's part."""
    bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return bits | ((int(phase) + 1) << 32)


def set_status_word(word: Optional[torch.Tensor]) -> None:
    """b200kv_set_status_word: register a device int32 word (or None) that collects the timeout bits of later launches."""
    check(lib.b200kv_set_status_word(None if word is None else word.data_ptr()), "b200kv_set_status_word")


STATUS_COPY_TIMEOUT, STATUS_SPLIT_TIMEOUT, STATUS_PEER_TIMEOUT, STATUS_PIPE_TIMEOUT = 1, 2, 4, 8


def workspace_reset(workspace: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
    check(lib.b200kv_workspace_reset(_ptr(workspace), workspace.numel() * workspace.element_size(), _stream(stream)), "b200kv_workspace_reset")


def set_decode_kernel(choice: int) -> None:
    """b200kv_set_decode_kernel: 0 = tcgen05 streaming kernel where it applies (default), 1 = warp-level mma kernel."""
    check(lib.b200kv_set_decode_kernel(int(choice)), "b200kv_set_decode_kernel")


def set_launch_overlap(tail_positions: int) -> None:
    """b200kv_set_launch_overlap: let consecutive append/decode kernels of a stream overlap (0 = off)."""
    check(lib.b200kv_set_launch_overlap(int(tail_positions)), "b200kv_set_launch_overlap")


def decode_kernel_kind(view: View, query_heads: int) -> int:
    """1: decode attention on this view runs a streaming int8 kernel (head_dim 128); 2: the tcgen05 stage 1 for head_dim 256;
    0: the generic kernel."""
    return int(lib.b200kv_decode_kernel_kind(C.byref(view), query_heads))


def _views(storages):
    return (View * len(storages))(*[st.view() for st in storages])


def save_session(path: str, model_id: str, quantization: str, prefix_tokens, storages,
                 stream: Optional[torch.cuda.Stream] = None) -> None:
    """PersistentSession::save_to_file (src/prefill_v2/persistent_session.cpp:34-142) for the attention layers."""
    toks = (C.c_uint32 * len(prefix_tokens))(*prefix_tokens)
    check(lib.b200kv_session_save(path.encode(), model_id.encode(), quantization.encode(), toks, len(prefix_tokens), _views(storages),
                                  len(storages), _stream(stream)), "b200kv_session_save")


def load_session(path: str, model_id: str, quantization: str, storages, stream: Optional[torch.cuda.Stream] = None):
    """PersistentSession::load_from_file (:168-267).  Returns the prefix tokens, or None when the file does not match
    or is damaged (the reference returns false); other errors raise."""
    cap = 1 << 20
    toks = (C.c_uint32 * cap)()
    n = C.c_uint32()
    rc = lib.b200kv_session_load(path.encode(), model_id.encode(), quantization.encode(), _views(storages), len(storages), toks, cap,
                                 C.byref(n), _stream(stream))
    if rc in (-7, -8, -9):
        return None
    check(rc, "b200kv_session_load")
    return list(toks[:n.value])


def find_matching_session(session_dir: str, model_id: str, quantization: str, prompt):
    """PersistentSession::find_matching_session (:269-320): (path, prefix_length) of the longest stored prefix, or None."""
    p = (C.c_uint32 * len(prompt))(*prompt)
    out = C.create_string_buffer(4096)
    n = C.c_uint32()
    rc = lib.b200kv_session_find(session_dir.encode(), model_id.encode(), quantization.encode(), p, len(prompt), out, 4096, C.byref(n))
    return (out.value.decode(), n.value) if rc == 0 else None


def _tokens(tokens):
    return (C.c_uint32 * len(tokens))(*tokens)


class SnapshotPool:
    """In-VRAM store of prefix snapshots with longest-prefix lookup (b200kv_pool_*): the KV part of the first
    engine's session checkpoints, tools/miinfer_cli.cpp:1043-1317 (radix tree over token ids, least-recently-used
    eviction, 8 entries / 3 GiB by default, captures only at multiples of `granularity` tokens)."""

    def __init__(self, model_id: str = "", quantization: str = "", *, max_entries: int = 8, max_bytes: int = 3 << 30, granularity: int = 512):
        self._h = C.c_void_p()
        self.model_id, self.quantization = model_id, quantization
        check(lib.b200kv_pool_create(C.byref(self._h), model_id.encode(), quantization.encode(), max_entries, max_bytes, granularity),
              "b200kv_pool_create")

    def close(self) -> None:
        if self._h:
            lib.b200kv_pool_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def capture(self, tokens, storages=None, *, index_only_bytes: Optional[int] = None, stream: Optional[torch.cuda.Stream] = None) -> bool:
        """Keep the first len(tokens) positions of every layer (or, with index_only_bytes, only the bookkeeping)."""
        done = C.c_int()
        if index_only_bytes is not None:
            check(lib.b200kv_pool_capture_index_only(self._h, _tokens(tokens), len(tokens), index_only_bytes, C.byref(done)),
                  "b200kv_pool_capture_index_only")
        else:
            check(lib.b200kv_pool_capture(self._h, _tokens(tokens), len(tokens), _views(storages), len(storages), _stream(stream), C.byref(done)),
                  "b200kv_pool_capture")
        return bool(done.value)

    def lookup(self, prompt, model_id: Optional[str] = None, quantization: Optional[str] = None):
        """(matched_length, common_length) of the longest stored proper prefix of `prompt`."""
        m, c = C.c_uint32(), C.c_uint32()
        check(lib.b200kv_pool_lookup(self._h, None if model_id is None else model_id.encode(),
                                     None if quantization is None else quantization.encode(), _tokens(prompt), len(prompt), C.byref(m), C.byref(c)),
              "b200kv_pool_lookup")
        return m.value, c.value

    def restore(self, prompt, storages, stream: Optional[torch.cuda.Stream] = None) -> int:
        """Copy the longest stored proper prefix of `prompt` into the caches; returns its length (0 = none)."""
        m = C.c_uint32()
        check(lib.b200kv_pool_restore(self._h, _tokens(prompt), len(prompt), _views(storages), len(storages), _stream(stream), C.byref(m)),
              "b200kv_pool_restore")
        return m.value

    def stats(self) -> dict:
        c = PoolCounters()
        check(lib.b200kv_pool_stats(self._h, C.byref(c)), "b200kv_pool_stats")
        return {n: getattr(c, n) for n, _ in PoolCounters._fields_}


class ReusableContext:
    """Prefix reuse around one set of layer caches: what PrefillV2Model::generate does with its ReusableContext and
    session directory (src/prefill_v2/model.cpp:751-775, 868-887).  `begin(prompt)` decides how much of the prompt is
    already covered -- the prefix resident in the caches, a pool snapshot, a session file, in that order -- and brings
    it into the caches; the caller prefills the rest and calls `commit(prompt)`."""

    LAYOUT_VERSION = 20260925

    def __init__(self, model_id: str, quantization: str, storages, *, pool: Optional[SnapshotPool] = None, enable_prefix_reuse: bool = True,
                 cache_prefix_after: bool = True, cache_prefix_len: int = 0, persistent_session_dir: str = ""):
        self.model_id, self.quantization, self.storages, self.pool = model_id, quantization, list(storages or []), pool
        self._dir = persistent_session_dir.encode()
        self.options = ReuseOptions(int(enable_prefix_reuse), int(cache_prefix_after), cache_prefix_len, self._dir)
        self.resident_tokens: list[int] = []

    def has_valid_prefix(self) -> bool:
        return len(self.resident_tokens) > 0

    def begin(self, prompt, stream: Optional[torch.cuda.Stream] = None) -> dict:
        stats = ReuseStats()
        views = _views(self.storages) if self.storages else None
        check(lib.b200kv_reuse_begin(C.byref(self.options), self.model_id.encode(), self.quantization.encode(), self.model_id.encode(),
                                     self.quantization.encode(), self.LAYOUT_VERSION, _tokens(self.resident_tokens), len(self.resident_tokens),
                                     self.pool._h if self.pool is not None else None, _tokens(prompt), len(prompt), views, len(self.storages),
                                     _stream(stream) if self.storages else None, C.byref(stats)), "b200kv_reuse_begin")
        out = {n: getattr(stats, n) for n, _ in ReuseStats._fields_}
        if stats.reuse_hit and stats.source != 1:
            self.resident_tokens = list(prompt[:stats.prefix_tokens_reused])
        elif not stats.reuse_hit:
            self.resident_tokens = []      # the caches are about to be overwritten from position 0
        return out

    def commit(self, prompt, stream: Optional[torch.cuda.Stream] = None) -> dict:
        cached, wrote = C.c_uint32(), C.c_int()
        views = _views(self.storages) if self.storages else None
        check(lib.b200kv_reuse_commit(C.byref(self.options), self.model_id.encode(), self.quantization.encode(),
                                      self.pool._h if self.pool is not None else None, _tokens(prompt), len(prompt), views, len(self.storages),
                                      _stream(stream) if self.storages else None, C.byref(cached), C.byref(wrote)), "b200kv_reuse_commit")
        if cached.value:
            self.resident_tokens = list(prompt[:cached.value])
        return {"cached_length": cached.value, "wrote_file": bool(wrote.value)}


def token_sequence_hash(tokens) -> int:
    arr = (C.c_uint32 * len(tokens))(*tokens)
    return int(lib.b200kv_token_sequence_hash(arr, len(tokens)))
