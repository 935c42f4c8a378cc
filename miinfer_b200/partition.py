"""Host-side partitioning of the KV path across the GPUs of one box.

The reference runs on one GPU; its design notes only sketch sharding by kv head
(docs/architecture.md:1035-1092).  Three partitions are used here:

* sessions  -> ranks, length-balanced (batched serving; no data-path collective);
* kv heads  -> ranks (no collective inside attention);
* positions -> ranks in contiguous, tile-aligned blocks (one long context); each
  rank produces one (m, l, acc) partial per query head and the partials are
  all-gathered and merged with the same log-sum-exp rule as the split-K stage 2
  (gfx906/kernels/qwen3_primitives.hip:2295-2352).

Pure Python (no CUDA): exercised on CPU with gloo in tests/test_partition_cpu.py.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

TILE = 32  # the streaming decode kernel works in tiles of 32 positions


def shard_range(length: int, rank: int, world: int, align: int = TILE) -> Tuple[int, int]:
    """Positions [begin, end) of `rank` when [0, length) is cut into `world` contiguous blocks
    whose boundaries are multiples of `align` (the last block takes the ragged tail)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    tiles = (length + align - 1) // align
    t0 = tiles * rank // world
    t1 = tiles * (rank + 1) // world
    return min(t0 * align, length), min(t1 * align, length)


def owner_of_position(position: int, length: int, world: int, align: int = TILE) -> int:
    """Rank whose shard holds `position` (where an appended token's K/V row goes)."""
    for r in range(world):
        b, e = shard_range(length, r, world, align)
        if b <= position < e:
            return r
    return world - 1


def partition_sessions(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time greedy bin packing of sessions by context length: returns, per rank,
    the indices of its sessions (each rank owns whole caches; outputs stay with the session)."""
    bins: List[List[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(len(lengths)), key=lambda j: (-lengths[j], j)):
        r = min(range(world), key=lambda k: (load[k], k))
        bins[r].append(i)
        load[r] += lengths[i]
    return [sorted(b) for b in bins]


def kv_head_range(kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
    if kv_heads % world:
        raise ValueError("kv heads must divide evenly over the ranks")
    per = kv_heads // world
    return rank * per, (rank + 1) * per


def pack_partial(m, l, acc):
    """One rank's partial as a single [query_heads, d + 2] tensor (one all-gather instead of three)."""
    import torch

    return torch.cat([m.unsqueeze(-1), l.unsqueeze(-1), acc], dim=-1).contiguous()


def unpack_partials(gathered):
    """[parts, query_heads, d + 2] -> (m [parts, H], l [parts, H], acc [parts, H, d]), contiguous."""
    return gathered[..., 0].contiguous(), gathered[..., 1].contiguous(), gathered[..., 2:].contiguous()


def all_gather_partials(dist, packed):
    """All-gather of the per-rank partials: the one exchange step of sequence-sharded decode
    (query_heads * (d + 2) fp32 per rank and layer)."""
    import torch

    world = dist.get_world_size()
    out = torch.empty((world * packed.shape[0],) + tuple(packed.shape[1:]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out, packed)   # concatenated along dim 0 (the form every backend accepts)
    return out.view((world,) + tuple(packed.shape))


def open_exchange(dist, query_heads: int, head_dim: int):
    """Set-up of the in-kernel cross-GPU merge of sequence-sharded decode: every rank creates its exchange
    buffer, the 64-byte handles are all-gathered (host objects, any backend) and every rank maps its peers'
    buffers.  Returns a `kv.Exchange`; call `.destroy()` after a barrier when done."""
    from . import kv

    world, rank = dist.get_world_size(), dist.get_rank()
    ex = kv.Exchange.create(query_heads, head_dim, world, rank)
    handles = [None] * world
    dist.all_gather_object(handles, ex.own_handle)
    ex.open_peers(handles)
    dist.barrier()
    return ex


def pick_batched_splits(lengths, kv_heads: int, cta_slots: int = 296, max_splits: int = 128) -> int:
    """Split count (of the longest session) for one batched decode launch over sessions of these lengths.
    A launch runs one CTA per (split, kv head, session) and `cta_slots` CTAs at a time (two per SM); the
    kernel gives a session one split per ceil(max_length / splits) positions (rounded up to 128).  The cost of
    a choice, in positions streamed per CTA slot, fitted to launches timed on a B200 (1, 2, 4 and 8-GPU shares
    of 80 sessions of 512..16384 positions):
      * up to two waves of CTAs the waves are what counts: waves x (positions per split + 2048, the fixed
        cost of a CTA: prologue, pipeline fill, merge of its warps, tagged partial);
      * beyond that the slots refill as CTAs retire, so the cost is (CTAs / slots) x (positions per split +
        3072), without rounding to whole waves.
    Among equally cheap choices the coarser one wins (fewer partials to merge).  The library's own default
    (one split per 2048 positions) ignores both the wave count and the fixed cost."""
    lengths = [int(x) for x in lengths if int(x) > 0]
    if not lengths:
        return 1
    longest = max(lengths)
    budget = max(1, min(max_splits, 1024 // max(1, len(lengths))))     # the library's split-slot budget
    best, best_cost = 1, None
    for splits in range(1, budget + 1):
        per = max(256, -(-(-(-longest // splits)) // 128) * 128)
        if -(-longest // per) > splits:      # rounding pushed the longest session over its split count
            continue
        ctas = sum(-(-n // per) for n in lengths) * kv_heads
        if ctas <= 2 * cta_slots:
            cost = -(-ctas // cta_slots) * (per + 2048)
        else:
            cost = ctas / cta_slots * (per + 3072)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    return best
