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


def pick_batched_plan(lengths, kv_heads: int, cta_slots: int = 296, max_splits: int = 128):
    """(num_splits, length_bound) for one batched decode launch over sessions of these lengths: pass them as
    `num_splits` and `max_length` of b200kv_decode_attn_batched.  The kernel gives a session one split (one CTA
    per kv head) per `ceil(length_bound / num_splits)` positions, rounded up to 128, and spreads the session's
    128-position tiles evenly over its splits; so the pair selects the positions per split, in steps of 128.
    The cost of a choice is the makespan of the launch as the hardware dispatches it: CTAs in block order (split
    fastest, then kv head, then session), each onto the slot that frees up first, a CTA holding its slot for
    (its tiles + 6) tile times -- the 6 stand for its prologue, pipeline fill, merge of its warps and tagged
    partial.  The makespan is averaged over the device's slot count (two per SM), 8 fewer and 16 fewer: launches
    that filled every slot measured 8 % slower than launches that left a few free (under launch overlap the next
    layer's first CTAs then have nowhere to start their ring fill), and a packing that only works out at one exact
    slot count does not survive the spread of real CTA times.  Fitted to launches timed on a B200 over 1-, 2-, 4-
    and 8-GPU shares of 80 sessions of 512..16384 positions (about a hundred split sizes in all): the model's
    choice is within 1.5 % of the measured best on average and 5 % at worst.  Equal costs go to the larger split
    (fewer partials).  The library's own default (one split per 2048 positions) ignores the slots.
    This is the pure-Python statement of b200kv_plan_batched_decode (csrc/plan.cpp), which a host calls instead (1 ms
    where this takes 0.1 s for 80 sessions); the tests hold the two against each other."""
    import heapq

    lengths = [int(x) for x in lengths if int(x) > 0]
    if not lengths:
        return 1, 0
    longest = max(lengths)
    budget = max(1, min(max_splits, 1024 // max(1, len(lengths))))     # the library's split-slot budget
    tiles = [-(-n // 128) for n in lengths]
    top = -(-longest // 128) * 128
    step = 128 * max(1, -(-top // (128 * 64)))                          # at most about 64 candidates
    best = None
    for per in range(max(256, step), top + step, step):
        splits = -(-longest // per)
        if splits > budget:
            continue
        durations = []
        for n, t in zip(lengths, tiles):
            k = -(-n // per)
            durations.extend([t * (c + 1) // k - t * c // k + 6 for c in range(k)] * kv_heads)
        cost = 0
        for slots in (cta_slots, cta_slots - 8, cta_slots - 16):
            free_at = [0] * max(1, slots)
            for d in durations:
                heapq.heapreplace(free_at, free_at[0] + d)
            cost += max(free_at)
        if best is None or cost <= best[0]:
            best = (cost, splits, splits * per)
    if best is None:                                                    # more sessions than the split budget serves
        return 1, longest
    return best[1], best[2]
