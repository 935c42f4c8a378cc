"""CPU tests of the multi-GPU host logic: partitioning, and the sequence-sharded merge run as two gloo
ranks against the oracle (each rank holds half of the positions; partials are all-gathered and merged)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_ranges_tile_and_cover():
    from miinfer_b200.partition import owner_of_position, shard_range

    for length in (1, 31, 32, 33, 4097, 131072, 131073):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(length, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == length
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 32 == 0 for b, _ in spans)
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 64 or length < 64 * world
            assert owner_of_position(length - 1, length, world) == max(r for r, (b, e) in enumerate(spans) if e > b)
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def test_session_partition_is_balanced_and_complete():
    from miinfer_b200.partition import kv_head_range, partition_sessions

    rng = np.random.default_rng(42)
    lengths = [int(x) for x in rng.integers(512, 16385, size=64)] + [4096] * 16
    for world in (1, 2, 4, 8):
        bins = partition_sessions(lengths, world)
        assert sorted(i for b in bins for i in b) == list(range(80))
        loads = [sum(lengths[i] for i in b) for b in bins]
        assert max(loads) <= 1.05 * sum(lengths) / world + max(lengths) / world
    assert kv_head_range(8, 3, 4) == (6, 8)
    with pytest.raises(ValueError):
        kv_head_range(8, 0, 3)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist

    import kvoracle as ko
    from miinfer_b200.partition import all_gather_partials, pack_partial, shard_range, unpack_partials

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)            # same seed on every rank: everyone can rebuild the full reference
    L, H, Hq, d = 1000, 2, 8, 128
    k = ko.normal_f16(rng, (L, H * d)).astype(np.float32); v = ko.normal_f16(rng, (L, H * d)).astype(np.float32)
    q = ko.normal_f16(rng, (Hq, d)).astype(np.float32)
    full = ko.HostCache(L, H, d, 32, 3); full.append(k, v, None, 0, rope_mode=0)
    ref, _ = full.decode_ref(q, d ** -0.5, L)
    b, e = shard_range(L, rank, world)
    shard = ko.HostCache(max(e - b, 1), H, d, 32, 3)      # this rank only holds its own positions
    if e > b:
        shard.append(k[b:e], v[b:e], None, 0, rope_mode=0)
    m, l, acc = shard.decode_partials(q, d ** -0.5, 0, e - b, 1)
    packed = pack_partial(torch.from_numpy(m[0]), torch.from_numpy(l[0]), torch.from_numpy(acc[0]))
    gathered = all_gather_partials(dist, packed)
    gm, gl, gacc = unpack_partials(gathered)
    out, _ = ko.merge_partials(gm.numpy(), gl.numpy(), gacc.numpy())
    err = float(np.max(np.abs(out - ref)))
    Path(tmp, f"rank{rank}.txt").write_text(repr(err))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharded_merge_over_gloo(tmp_path, world):
    import torch.multiprocessing as mp

    port = 29500 + os.getpid() % 1000 + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float((tmp_path / f"rank{r}.txt").read_text()) <= 2e-6


def test_pick_batched_plan_packs_the_slots_and_respects_budgets():
    from miinfer_b200.partition import partition_sessions, pick_batched_plan

    def per_split(splits, bound):          # what the library derives from the pair
        return max(256, -(-(-(-bound // splits)) // 128) * 128)

    rng = np.random.default_rng(42)
    lengths = [int(x) for x in rng.integers(512, 16385, size=10)]
    splits, bound = pick_batched_plan(lengths, 8)
    per = per_split(splits, bound)
    # the bound covers every session, the longest session fits its split count, and the launch is one wave
    assert bound >= max(lengths) and -(-max(lengths) // per) <= splits
    assert sum(-(-n // per) for n in lengths) * 8 <= 296
    # the bench's 80 sessions: the split sizes that timed best (or within 2 % of it) on the device for a 1-, 2-, 4-
    # and 8-GPU share
    all_lengths = [int(x) for x in np.random.default_rng(42).integers(512, 16385, size=64)] + [4096] * 16
    for world, want in ((1, (7168,)), (2, (6144,)), (4, (2816,)), (8, (2560, 2688, 2816))):
        for share in partition_sessions(all_lengths, world):
            s, b = pick_batched_plan([all_lengths[i] for i in share], 8)
            assert per_split(s, b) in want
    # a single short session needs one split; many sessions are capped by the split-slot budget (1024 slots)
    assert pick_batched_plan([100], 8)[0] == 1
    assert pick_batched_plan([16384] * 256, 8)[0] <= 4
    assert pick_batched_plan([], 8)[0] == 1
    assert pick_batched_plan([0, 0], 8)[0] == 1


def test_native_batched_plan_equals_the_python_statement():
    """b200kv_plan_batched_decode is host arithmetic: callable without a GPU.  Same pair as partition.pick_batched_plan
    for mixed, uniform, tiny, empty and over-budget session sets, and for another slot count."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import pick_batched_plan

    rng = np.random.default_rng(5)
    cases = [[int(x) for x in rng.integers(1, 20000, size=n)] for n in (1, 3, 10, 40, 80, 200)]
    cases += [[4096] * 16, [100], [], [0, 0], [16384] * 256, [131072], [300, 0, 70000]]
    for lengths in cases:
        for kv_heads, slots in ((8, 296), (4, 296), (8, 264)):
            assert kv.plan_batched_decode(lengths, kv_heads, slots) == pick_batched_plan(lengths, kv_heads, cta_slots=slots), (lengths[:4], kv_heads, slots)
    assert kv.plan_batched_decode([5000, 9000], 8) == kv.plan_batched_decode([5000, 9000], 8, 296)     # 0 = the B200 default
