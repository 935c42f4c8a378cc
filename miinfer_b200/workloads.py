"""Secondary bench workloads: suffix prefill (a 512-token chunk over an 8192-token q8_0 prefix), batched serving
(64 sessions of mixed length plus 16 restored from a shared prefix snapshot) and sequence-sharded long-context
decode (one 131072-token session over the ranks).  bench.py dispatches here for --workload prefill|batched|seqshard,
and calls `extras` to attach them as sub-records to its default line.  Every workload function can be run with
`dist=None, world=1` inside a multi-rank job (rank 0 does that to measure a workload's own 1-GPU time), and every
one ends with a comparison of one layer's output against the CPU oracle evaluated on the cache planes as they lie on
the device (`check`): test infrastructure used as the checker, outside every timed region."""
from __future__ import annotations

import json
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def _peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


def _oracle():
    tests = str(ROOT / "tests")
    if tests not in sys.path:
        sys.path.insert(0, tests)
    import kvoracle as ko

    return ko


def host_cache_from_planes(ko, planes: dict, capacity: int, kv_heads: int, head_dim: int, qblock: int = 32):
    """An oracle-side cache over numpy copies of device planes (int8 K/V, fp16 scales as uint16)."""
    host = ko.HostCache(capacity, kv_heads, head_dim, qblock, 3)
    host.key_q8[...] = planes["key_q8"]
    host.value_q8[...] = planes["value_q8"]
    host.key_scales[...] = planes["key_scales"]
    host.value_scales[...] = planes["value_scales"]
    return host


def planes_of(torch, storage, rows: int) -> dict:
    """The first `rows` positions of a Q8/Q8 storage object's planes as numpy arrays."""
    return {"key_q8": storage.key_cache_q8[:, :rows].cpu().numpy(), "value_q8": storage.value_cache_q8[:, :rows].cpu().numpy(),
            "key_scales": storage.key_scales[:, :rows].contiguous().view(torch.int16).cpu().numpy().view(np.uint16),
            "value_scales": storage.value_scales[:, :rows].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)}


def error_record(got: np.ndarray, ref: np.ndarray, **extra) -> dict:
    diff = got.astype(np.float64) - ref.astype(np.float64)
    rec = {"max_abs": float(np.max(np.abs(diff))), "rel_l2": float(np.linalg.norm(diff) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)),
           "against": "CPU oracle (two-pass fp32 softmax) on the device's cache planes", "tolerance_max_abs": 2.0e-3}
    rec["ok"] = bool(np.isfinite(got).all() and rec["max_abs"] <= 2.0e-3)
    rec.update(extra)
    return rec


def _fill(kv, torch, st, tokens, seed, chunk=8192):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    width = st.kv_heads * st.head_dim
    for base in range(0, tokens, chunk):
        n = min(chunk, tokens - base)
        k = torch.randn(n, width, generator=g, device="cuda").half()
        v = torch.randn(n, width, generator=g, device="cuda").half()
        kv.launch_kv_store_quant(st.view(), k, v, None, n, base, rope_mode=kv.RopeMode.NONE)


def _time(torch, dist, stream, fn, warmup, steps):
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def run_prefill(args, torch, dist, rank, world, local_rank):
    """512-token chunk appended to an 8192-token q8_0 prefix, 24 Q / 4 KV heads, d=256, 16 layers.
    With N GPUs the 4 kv heads (and their 6 query heads each) are split over the ranks."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import kv_head_range

    P, T, HQ, HKV, D, LAYERS = 8192, 512, 24, 4, 256, min(args.layers, 16)
    h0, h1 = kv_head_range(HKV, rank, world)
    hkv, hq = h1 - h0, (h1 - h0) * (HQ // HKV)
    caches = [kv.AttentionLayerKvCacheStorage(P + T, kv.KvCacheQuantMode.kQ8Q8, kv_heads=hkv, head_dim=D, qblock=32) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        _fill(kv, torch, c, P, 100 * rank + i)
    g = torch.Generator(device="cuda"); g.manual_seed(7 + rank)
    q = torch.randn(LAYERS, T, hq, D, generator=g, device="cuda").half()
    gate = torch.randn(LAYERS, T, hq, D, generator=g, device="cuda")
    k_new = torch.randn(LAYERS, T, hkv * D, generator=g, device="cuda").half()
    v_new = torch.randn(LAYERS, T, hkv * D, generator=g, device="cuda").half()
    w = torch.ones(D, device="cuda")
    out = torch.zeros(LAYERS, T, hq, D, device="cuda")
    views = [c.view() for c in caches]
    # the fp16 scratch of the visible prefix selects the tcgen05 kernel; --prefill-kernel mma runs the mma.sync one
    # (with room for KV-split partials: the chunk's row tiles alone do not fill the SMs)
    ws = None if args.prefill_kernel == "mma" else kv.prefill_workspace(P + T, hkv, D, token_count=T, query_heads=hq)
    # The fp16 copy of a layer's prefix does not depend on the chunk: with a second workspace and a second stream the
    # pre-pass of layer l + 1 runs beside the attention of layer l; a layer's own launch then converts only its chunk.
    # (Not with one kv head per GPU: a layer then takes about 50 us, which the extra stream and event calls of this eager
    # loop exceed on the host -- 0.92 ms per chunk against 0.80.)
    ahead = ws is not None and not getattr(args, "no_prepare_ahead", False) and LAYERS >= 2 and hkv >= 2
    ws2 = kv.prefill_workspace(P + T, hkv, D, token_count=T, query_heads=hq) if ahead else None
    stream = torch.cuda.Stream()
    side = torch.cuda.Stream() if ahead else None
    attended = [torch.cuda.Event() for _ in range(LAYERS)] if ahead else None
    prepared = [torch.cuda.Event() for _ in range(LAYERS)] if ahead else None

    def prepare(l):
        side.wait_event(attended[l - 2]) if l >= 2 else side.wait_stream(stream)   # the workspace's previous user
        kv.prepare_suffix_attention(views[l], P, P + T, ws2 if l & 1 else ws, stream=side)
        prepared[l].record(side)

    def step():
        if ahead:
            prepare(0)
            prepare(1)
        for l in range(LAYERS):
            kv.launch_kv_store_quant(views[l], k_new[l], v_new[l], w, T, P, rope_mode=kv.RopeMode.SECTIONED64, theta=1.0e6)
            if ahead:
                stream.wait_event(prepared[l])
                kv.launch_suffix_attention_quant(views[l], q[l], gate[l], out[l], ws2 if l & 1 else ws, T, P, query_heads=hq,
                                                 scale=D ** -0.5, prepared_rows=P)
                attended[l].record(stream)
                if l + 2 < LAYERS:
                    prepare(l + 2)
            else:
                kv.launch_suffix_attention_quant(views[l], q[l], gate[l], out[l], ws, T, P, query_heads=hq, scale=D ** -0.5)
        if ahead:
            stream.wait_stream(side)

    kv.set_launch_overlap(0 if args.no_overlap else 1)   # every kernel of the chunk waits for its predecessor itself
    ms = _time(torch, dist, stream, step, args.warmup, args.steps)
    kv.set_launch_overlap(0)
    check = None
    if rank == 0 and not args.no_check:
        ko = _oracle()
        ko.set_threads(args.cpu_threads)
        host = host_cache_from_planes(ko, planes_of(torch, caches[0], P + T), P + T, hkv, D)
        tokens = 64     # the last 64 query tokens of the chunk see the longest ranges; the oracle costs ~14 ms per token
        ref = host.suffix_ref(q[0, T - tokens:].float().cpu().numpy(), gate[0, T - tokens:].cpu().numpy(), P + T - tokens, D ** -0.5)
        check = error_record(out[0, T - tokens:].cpu().numpy(), ref, layer=0, tokens=f"last {tokens} of {T}")
    flops = 4.0 * D * HQ * (T * P + T * (T + 1) / 2) * LAYERS   # QK^T and PV over the causal ranges, all heads
    _, tf_peak, kind = _peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    return {"metric": "suffix_prefill_tflops_512_over_8192", "value": achieved, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 KV dequantised to fp16, fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"prefill: {T}-token chunk over {P}-token q8_0 prefix, {HQ} Q / {HKV} KV heads, d={D}, {LAYERS} layers; "
                                   f"kv heads split over {world} GPU(s); kernel {args.prefill_kernel}", "l2": "L2 flushed implicitly: 16 layer caches of 19 MB rotate"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak * world, "unit": "TFLOP/s", "frac": achieved / (tf_peak * world),
                         "traffic": None, "peak_kind": f"{kind} (bf16_tflops_sustained) x {world} GPUs"},
            "check": check, "gpu_launches": args.steps * LAYERS * (2 if ws is None else (5 if ahead else 4)),
            "prefix_prepass": "beside the previous layers' attention (second stream, two workspaces)" if ahead else "inside the layer's own launch sequence"}


def run_seqshard(args, torch, dist, rank, world, local_rank):
    """One 131072-token session, KV sharded by position over the ranks.  Per layer each rank reduces its shard to one
    (m, l, acc) partial per query head; with `--exchange kernel` (default) the decode kernel itself stores that
    partial into every peer's exchange buffer over NVLink and merges what it receives, with `--exchange nccl` the
    partials are all-gathered by NCCL and merged by a second kernel."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import open_exchange, shard_range

    L, HQ, HKV, D, LAYERS = args.seq_context, 32, 8, 128, args.layers
    b, e = shard_range(L, rank, world)
    n = e - b
    cap = (n + 64 + 63) // 64 * 64
    caches = [kv.AttentionLayerKvCacheStorage(cap, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=32) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        _fill(kv, torch, c, n, 1000 * rank + i)
    g = torch.Generator(device="cuda"); g.manual_seed(99)
    q = torch.randn(LAYERS, HQ, D, generator=g, device="cuda").half()      # replicated query (same seed on every rank)
    out = torch.zeros(LAYERS, HQ, D, device="cuda")
    mine = kv.packed_partial(HQ, D, 1)                 # this rank's (m | l | acc), written in place by the kernel
    pm, pl, pa = kv.partial_views(mine[0], HQ, D)
    gathered = kv.packed_partial(HQ, D, world)
    ws = kv.decode_workspace(HQ, D)
    views = [c.view() for c in caches]
    in_kernel = dist is not None and getattr(args, "exchange", "kernel") == "kernel"
    nccl_c = dist is not None and getattr(args, "exchange", "kernel") == "nccl-c"
    exchange = open_exchange(dist, HQ, D) if in_kernel else None
    dm = None
    if nccl_c:   # the library's own NCCL communicator (b200kv_dist_*), its unique id handed round through torch.distributed
        ids = [kv.DistMerge.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        dm = kv.DistMerge(ids[0], rank, world, HQ, D)
    kv.set_launch_overlap(0 if (args.no_overlap or (dist is not None and not in_kernel)) else 1)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kv.set_status_word(status)

    def step():
        for l in range(LAYERS):
            if dist is None:
                kv.launch_decode_attention_quant(views[l], q[l], query_heads=HQ, scale=D ** -0.5, cache_length=n, output=out[l], workspace=ws)
                continue
            if in_kernel:
                # the call number on this exchange: consecutive layers alternate the slot, and the step's second half
                # continues the count so that a replayed graph never meets its own previous words in the same slot
                kv.launch_decode_attention_sharded(views[l], q[l], exchange, query_heads=HQ, scale=D ** -0.5, range_begin=0,
                                                   range_end=n, phase=l, output=out[l], workspace=ws)
                continue
            if nccl_c:
                dm.decode_partials(views[l], q[l], scale=D ** -0.5, range_begin=0, range_end=n, workspace=ws)
                dm.merge(output=out[l])
                continue
            kv.launch_decode_partials(views[l], q[l], query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=n,
                                      part_m=pm, part_l=pl, part_acc=pa, workspace=ws)
            dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))     # 16.6 KB per rank: the one exchange step
            kv.launch_merge_partials_packed(gathered, num_parts=world, query_heads=HQ, head_dim=D, output=out[l])

    if in_kernel and LAYERS % 2:
        raise SystemExit("seqshard --exchange kernel alternates two exchange slots per layer: use an even --layers")
    # the whole decode step (kernels and collectives) is captured once and replayed: the exchange is latency-bound
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
    torch.cuda.synchronize()
    ms = _time(torch, dist, stream, graph.replay, args.warmup, args.steps)
    kv.set_status_word(None)
    kv.set_launch_overlap(0)
    checksum = float(out.double().abs().sum().item())   # identical on every rank when the exchange is right
    checksum_spread = 0.0
    check = None
    if dist is not None:
        sums = [None] * world
        dist.all_gather_object(sums, checksum)
        checksum_spread = (max(sums) - min(sums)) / max(abs(max(sums)), 1e-30)
    if not args.no_check:
        # layer 0 against the oracle over the WHOLE context: every rank's shard of layer 0 is gathered to rank 0
        p = planes_of(torch, caches[0], n)
        flat = torch.cat([torch.from_numpy(p[k].reshape(-1).view(np.uint8)) for k in ("key_q8", "value_q8", "key_scales", "value_scales")]).cuda()
        if dist is not None:
            sizes = [None] * world
            dist.all_gather_object(sizes, int(n))
            if len(set(sizes)) != 1:
                flat = None     # ragged shards: the gather below assumes equal ones
            else:
                allp = torch.empty(world * flat.numel(), dtype=torch.uint8, device="cuda")
                dist.all_gather_into_tensor(allp, flat)
                flat = allp
        if rank == 0 and flat is not None:
            ko = _oracle()
            ko.set_threads(args.cpu_threads)
            host = ko.HostCache(L, HKV, D, 32, 3)
            per = flat.numel() // world
            for r in range(world):
                rb, re_ = shard_range(L, r, world)
                m = re_ - rb
                blob = flat[r * per:(r + 1) * per].cpu().numpy()
                o = 0
                for name, width, dt in (("key_q8", D, np.int8), ("value_q8", D, np.int8), ("key_scales", 8, np.uint16), ("value_scales", 8, np.uint16)):
                    nbytes = HKV * m * width
                    arr = blob[o:o + nbytes].view(dt).reshape(HKV, m, -1)
                    getattr(host, name)[:, rb:re_] = arr
                    o += nbytes
            ref, _ = host.decode_ref(q[0].float().cpu().numpy(), D ** -0.5, L)
            check = error_record(out[0].cpu().numpy(), ref, layer=0, context=L,
                                 exchange=("in-kernel peer stores" if in_kernel else "NCCL all-gather") if dist is not None else "none (1 GPU)")
    if exchange is not None:
        dist.barrier()
        exchange.destroy()
    if dm is not None:
        # NCCL's communicator teardown waits for every CUDA graph that captured one of its collectives to be destroyed
        graph.reset()
        del graph
        dist.barrier()
        dm.destroy()
    bw_peak, _, kind = _peaks()
    bytes_total = LAYERS * L * HKV * 136 * 2
    achieved = bytes_total / (ms * 1e-3) / 1e9
    return {"metric": "q8_0_kv_decode_tokens_per_s_128k_ctx_sequence_sharded", "value": 1000.0 / ms, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"seqshard: one {L}-token session, {LAYERS} layers, {HQ} Q / {HKV} KV heads, d={D}, q8_0; positions sharded over "
                                   f"{world} GPU(s); per layer exchange of {HQ}x({D}+2) fp32 per rank "
                                   f"({'peer stores + merge inside the decode kernel' if in_kernel else ('NCCL all-gather + merge kernel through the C entry points' if nccl_c else 'NCCL all-gather + merge kernel')})",
                       "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak * world, "unit": "GB/s", "frac": achieved / (bw_peak * world),
                         "traffic": None, "peak_kind": f"{kind} x {world} GPUs"},
            "merge_bytes_per_layer_per_rank": HQ * (D + 2) * 4, "output_checksum": checksum, "output_checksum_spread_over_ranks": checksum_spread,
            "status_word": int(status.item()), "check": check,
            "gpu_launches": args.steps * LAYERS * (1 if (dist is None or in_kernel) else 3)}


def run_batched(args, torch, dist, rank, world, local_rank):
    """64 sessions with context lengths uniform in [512, 16384] (seeded), one decode step each per layer in ONE launch,
    plus 16 sessions restored from a shared 4096-token prefix snapshot kept in a snapshot pool; sessions are bin-packed
    over the ranks."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import partition_sessions

    HQ, HKV, D, LAYERS = 32, 8, 128, min(args.layers, 4)
    rng = np.random.default_rng(42)
    lengths_all = [int(x) for x in rng.integers(512, 16385, size=64)] + [4096] * 16
    mine = partition_sessions(lengths_all, world)[rank]
    lengths = [lengths_all[i] for i in mine]
    restored = [i for i in mine if i >= 64]
    caches = [[kv.AttentionLayerKvCacheStorage((L + 8 + 63) // 64 * 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=32)
               for L in lengths] for _ in range(LAYERS)]
    proto = [kv.AttentionLayerKvCacheStorage(4096 + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=32) for _ in range(LAYERS)]
    for l in range(LAYERS):
        _fill(kv, torch, proto[l], 4096, 5000 + l)
        for j, (i, L) in enumerate(zip(mine, lengths)):
            if i < 64:
                _fill(kv, torch, caches[l][j], L, 10000 * l + i)
    # the shared prefix lives in an in-VRAM snapshot pool under its token ids; restored sessions look it up
    prefix_tokens = [int(t) for t in np.random.default_rng(7).integers(0, 150000, 4096)]
    pool = kv.SnapshotPool(max_entries=8, max_bytes=3 << 30)
    pool.capture(prefix_tokens, proto)
    S = len(mine)
    g = torch.Generator(device="cuda"); g.manual_seed(rank)
    q = torch.randn(LAYERS, S, HQ, D, generator=g, device="cuda").half()
    out = torch.zeros(LAYERS, S, HQ, D, device="cuda")
    lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ws = kv.decode_workspace(HQ, D, S)
    tables = [kv.view_table(S) for _ in range(LAYERS)]
    stream = torch.cuda.current_stream()

    # restore of the snapshot sessions: longest-prefix lookup in the pool, then a device-to-device clone of the
    # matched 4096 positions per layer; timed on its own
    def restore():
        for j, i in enumerate(mine):
            if i >= 64:
                matched = pool.restore(prefix_tokens + [1, 2, 3], [caches[l][j] for l in range(LAYERS)])
                assert matched == 4096
    restore_ms = _time(torch, dist, stream, restore, 1, 3) if restored or dist is not None else 0.0
    # the host knows this step's lengths: pick the split size whose CTAs pack the device best (0 = library default)
    splits, bound = (0, max(lengths)) if getattr(args, "default_splits", False) else kv.plan_batched_decode(lengths, HKV)
    kv.set_launch_overlap(0 if args.no_overlap else 1)
    for l in range(LAYERS):   # fills the device view tables once
        kv.launch_decode_attention_batched([c.view() for c in caches[l]], tables[l], lens, bound, q[l], query_heads=HQ,
                                           scale=D ** -0.5, output=out[l], workspace=ws, num_splits=splits)

    def step():
        for l in range(LAYERS):
            kv.launch_decode_attention_batched(None, tables[l], lens, bound, q[l], query_heads=HQ, scale=D ** -0.5,
                                               output=out[l], workspace=ws, num_splits=splits)

    # the step is captured once and replayed (the launches are asynchronous: the table's geometry is remembered on the host)
    gstream = torch.cuda.Stream()
    with torch.cuda.stream(gstream):
        step()
        gstream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=gstream):
            step()
    torch.cuda.synchronize()
    ms = _time(torch, dist, gstream, graph.replay, args.warmup, args.steps)
    kv.set_launch_overlap(0)
    check = None
    if rank == 0 and not args.no_check:
        ko = _oracle()
        ko.set_threads(args.cpu_threads)
        worst = {"max_abs": 0.0, "rel_l2": 0.0}
        picks = [0, S - 1] + ([mine.index(restored[0])] if restored else [])     # the longest, the shortest and a restored session
        for j in picks:
            host = host_cache_from_planes(ko, planes_of(torch, caches[0][j], lengths[j]), lengths[j], HKV, D)
            ref, _ = host.decode_ref(q[0, j].float().cpu().numpy(), D ** -0.5, lengths[j])
            rec = error_record(out[0, j].cpu().numpy(), ref)
            worst = {k: max(worst[k], rec[k]) for k in worst}
        check = {**worst, "ok": bool(worst["max_abs"] <= 2.0e-3), "layer": 0, "sessions_checked": len(picks),
                 "against": "CPU oracle (two-pass fp32 softmax) on the device's cache planes", "tolerance_max_abs": 2.0e-3}
    bw_peak, _, kind = _peaks()
    bytes_total = LAYERS * sum(lengths_all) * HKV * 136 * 2
    achieved = bytes_total / (ms * 1e-3) / 1e9
    return {"metric": "batched_decode_session_steps_per_s", "value": len(lengths_all) * 1000.0 / ms, "unit": f"session-steps/s over {LAYERS} layers",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"batched: 64 sessions U[512,16384] + 16 restored from a 4096-token snapshot, {LAYERS} layers, {HQ} Q / {HKV} KV, d={D}, "
                                   f"q8_0; sessions bin-packed over {world} GPU(s)", "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak * world, "unit": "GB/s", "frac": achieved / (bw_peak * world),
                         "traffic": None, "peak_kind": f"{kind} x {world} GPUs"},
            "splits_of_longest_session": splits, "positions_per_split": (bound // splits if splits else 2048), "restore_ms_16_sessions": restore_ms, "restore_bytes": LAYERS * 16 * 4096 * HKV * 136 * 2,
            "check": check, "gpu_launches": args.steps * LAYERS}


def run_append(args, torch, dist, rank, world, local_rank):
    """The store kernel alone (K-norm, RoPE, q8_0 quantisation, cache write): `--append-tokens` fp16 rows per layer
    into `--layers` caches.  Default 8192 tokens x 8 kv heads x d=128 with NeoX RoPE (a prefill chunk of the decode
    benchmark's model); `--append-shape chunk256` is the 512-token chunk of the 24 Q / 4 KV d=256 model with the
    sectioned RoPE.  Every layer has its own inputs and cache, so a step streams more than L2 holds."""
    from miinfer_b200 import kv

    if args.append_shape == "chunk256":
        T, HKV, D, mode, LAYERS = 512, 4, 256, kv.RopeMode.SECTIONED64, max(args.layers, 36)
    else:
        T, HKV, D, mode, LAYERS = args.append_tokens, 8, 128, kv.RopeMode.NEOX_FULL, args.layers
    caches = [kv.AttentionLayerKvCacheStorage(T, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=32) for _ in range(LAYERS)]
    g = torch.Generator(device="cuda"); g.manual_seed(5 + rank)
    k_new = torch.randn(LAYERS, T, HKV * D, generator=g, device="cuda").half()
    v_new = torch.randn(LAYERS, T, HKV * D, generator=g, device="cuda").half()
    w = (1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")).float()
    views = [c.view() for c in caches]

    def step():
        for l in range(LAYERS):
            kv.launch_kv_store_quant(views[l], k_new[l], v_new[l], w, T, 0, rope_mode=mode, theta=1.0e6)

    # the launches are captured once and replayed, so short launches are timed on the device, not on the host's launch rate
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
    torch.cuda.synchronize()
    ms = _time(torch, dist, stream, graph.replay, args.warmup, args.steps)
    check = None
    if rank == 0 and not args.no_check:
        ko = _oracle()
        ko.set_threads(args.cpu_threads)
        rows = min(T, 512)
        host = ko.HostCache(rows, HKV, D, 32, 3)
        host.append(k_new[0, :rows].float().cpu().numpy(), v_new[0, :rows].float().cpu().numpy(), w.cpu().numpy(), 0, rope_mode=int(mode), theta=1.0e6)
        got = planes_of(torch, caches[0], rows)
        same = all(np.array_equal(got[k], getattr(host, k)[:, :rows]) for k in ("key_q8", "value_q8", "key_scales", "value_scales"))
        check = {"bit_exact": bool(same), "ok": bool(same), "rows": rows, "layer": 0, "against": "CPU oracle store (same quantiser, pinned trigonometry)"}
    row_out = D + 2 * (D // 32)
    bytes_step = LAYERS * T * HKV * 2 * (D * 2 + row_out)
    bw_peak, _, kind = _peaks()
    achieved = bytes_step / (ms * 1e-3) / 1e9
    return {"metric": "kv_append_gbs", "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 in, int8 + fp16 scales out",
            "data": "synthetic",
            "config": {"workload": f"append: {T} tokens x {HKV} kv heads x d={D} per layer, {LAYERS} layers, K-norm + {mode.name} RoPE + q8_0 store",
                       "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB per step"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak, "unit": "GB/s", "frac": achieved / bw_peak, "traffic": None,
                         "peak_kind": f"{kind} (hbm_gbs)", "kernel": "append_kernel", "us_per_launch": ms * 1e3 / LAYERS,
                         "algorithmic_bytes_per_launch": bytes_step // LAYERS},
            "check": check, "gpu_launches": args.steps * LAYERS}


def run_decode256(args, torch, dist, rank, world, local_rank):
    """Decode attention alone on the reference's own geometry: 24 query heads over 4 kv heads, head_dim 256, q8_0 K/V, one
    session of `--context` positions per GPU, 16 attention layers (the hybrid model's count), no append.  Stage 1 on the
    tcgen05 kernel for head_dim 256 plus the merge kernel; `--decode-kernel mma` runs the generic stage 1 instead."""
    from miinfer_b200 import kv

    L, HQ, HKV, D, LAYERS = args.context, 24, 4, 256, min(args.layers, 16)
    cap = (L + 64 + 127) // 128 * 128
    caches = [kv.AttentionLayerKvCacheStorage(cap, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=32) for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        _fill(kv, torch, c, L, 500 * rank + i)
    g = torch.Generator(device="cuda"); g.manual_seed(3 + rank)
    q = torch.randn(LAYERS, HQ, D, generator=g, device="cuda").half()
    out = torch.zeros(LAYERS, HQ, D, device="cuda")
    ws = kv.decode_workspace(HQ, D)
    views = [c.view() for c in caches]
    kind = kv.decode_kernel_kind(views[0], HQ)
    kv.set_launch_overlap(0 if args.no_overlap else 1)

    def step():
        for l in range(LAYERS):
            kv.launch_decode_attention_quant(views[l], q[l], query_heads=HQ, scale=D ** -0.5, cache_length=L, output=out[l], workspace=ws)

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
    torch.cuda.synchronize()
    ms = _time(torch, dist, stream, graph.replay, args.warmup, args.steps)
    kv.set_launch_overlap(0)
    check = None
    if rank == 0 and not args.no_check:
        ko = _oracle()
        ko.set_threads(args.cpu_threads)
        host = host_cache_from_planes(ko, planes_of(torch, caches[0], L), L, HKV, D)
        ref, _ = host.decode_ref(q[0].float().cpu().numpy(), D ** -0.5, L)
        check = error_record(out[0].cpu().numpy(), ref, layer=0, context=L)
    bytes_launch = L * HKV * (D + 2 * (D // 32)) * 2
    bw_peak, _, kind_peak = _peaks()
    achieved = bytes_launch * LAYERS / (ms * 1e-3) / 1e9
    streaming = kind == 2 and args.decode_kernel != "mma"
    return {"metric": "q8_0_kv_decode_attention_gbs_head_dim_256", "value": achieved * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"decode256: decode attention, {HQ} Q / {HKV} KV heads, d={D}, q8_0 K/V, context {L}, {LAYERS} layers, batch 1 per GPU",
                       "l2": f"inputs larger than L2: {bytes_launch * LAYERS / 1e6:.0f} MB of KV per step"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak, "unit": "GB/s", "frac": achieved / bw_peak, "traffic": None,
                         "peak_kind": f"{kind_peak} (hbm_gbs)",
                         "kernel": "decode_tc5_wide_kernel + merge_kernel" if streaming else "decode_generic_kernel + merge_kernel",
                         "us_per_launch_pair": ms * 1e3 / LAYERS, "algorithmic_bytes_per_launch": bytes_launch},
            "check": check, "gpu_launches": args.steps * LAYERS * 2}


def run(args, torch, dist, rank, world, local_rank):
    fn = {"prefill": run_prefill, "seqshard": run_seqshard, "batched": run_batched, "append": run_append, "decode256": run_decode256}.get(args.workload)
    if fn is None:
        raise SystemExit(f"unknown workload {args.workload}")
    line = fn(args, torch, dist, rank, world, local_rank)
    return line if rank == 0 else None


def _brief(line: dict, base: dict | None = None) -> dict:
    keep = {k: line[k] for k in ("metric", "value", "unit", "ms_per_step", "scaling", "n_gpus", "steps", "warmup", "roofline", "check",
                                 "gpu_launches") if k in line}
    keep["workload"] = line["config"]["workload"]
    for k in ("restore_ms_16_sessions", "splits_of_longest_session", "positions_per_split", "output_checksum_spread_over_ranks", "status_word"):
        if k in line:
            keep[k] = line[k]
    if base is not None:
        keep["single_gpu_ms_per_step"] = base["ms_per_step"]
        keep["single_gpu_source"] = "measured in this run on rank 0 alone, same problem, same kernels"
        keep["speedup_over_single_gpu"] = base["ms_per_step"] / line["ms_per_step"]
    return keep


def extras(args, torch, dist, rank, world, local_rank) -> dict:
    """Sub-records for bench.py's default line: `prefill` always; on one GPU also `decode256` and `append`; with N > 1 GPUs
    `seqshard` and `batched`, each next to its own 1-GPU time measured by rank 0 alone on the full problem while the other
    ranks wait on the host."""
    sub = SimpleNamespace(**vars(args))
    sub.steps, sub.warmup = max(3, min(args.steps, 20)), 3
    out = {}

    def release():
        import gc
        gc.collect()
        torch.cuda.empty_cache()

    def alone(fn):
        """rank 0 runs `fn` as a 1-GPU job; the others block on the host (a store key, not a GPU-side barrier)."""
        res = None
        if rank == 0:
            res = fn(sub, torch, None, 0, 1, local_rank)
            release()
        if dist is not None:
            store = dist.distributed_c10d._get_default_store()
            key = f"alone_{fn.__name__}"
            if rank == 0:
                store.set(key, "done")
            else:
                store.wait([key])
            dist.barrier()
        return res

    if world in (1, 2, 4):
        line = run_prefill(sub, torch, dist, rank, world, local_rank)
        release()
        base = alone(run_prefill) if world > 1 else None
        if rank == 0:
            out["prefill"] = _brief(line, base)
    if world == 1:
        # the reference's own decode geometry (24 Q / 4 KV, head_dim 256) at the headline context, and the store kernel alone
        d256 = SimpleNamespace(**vars(sub))
        d256.context = 32768
        out["decode256"] = _brief(run_decode256(d256, torch, None, 0, 1, local_rank))
        release()
        out["append"] = _brief(run_append(sub, torch, None, 0, 1, local_rank))
        release()
    if world > 1:
        for name, fn in (("seqshard", run_seqshard), ("batched", run_batched)):
            line = fn(sub, torch, dist, rank, world, local_rank)
            release()
            base = alone(fn)
            if rank == 0:
                out[name] = _brief(line, base)
    return out
