"""Secondary bench workloads: suffix prefill (BASELINE config 3), batched
serving (config 4) and sequence-sharded long-context decode (config 5).  bench.py dispatches here
for --workload prefill|batched|seqshard; the default decode32k workload lives in bench.py."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def _peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


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

    def step():
        for l in range(LAYERS):
            kv.launch_kv_store_quant(views[l], k_new[l], v_new[l], w, T, P, rope_mode=kv.RopeMode.SECTIONED64, theta=1.0e6)
            kv.launch_suffix_attention_quant(views[l], q[l], gate[l], out[l], ws, T, P, query_heads=hq, scale=D ** -0.5)

    stream = torch.cuda.Stream()
    ms = _time(torch, dist, stream, step, args.warmup, args.steps)
    flops = 4.0 * D * HQ * (T * P + T * (T + 1) / 2) * LAYERS   # QK^T and PV over the causal ranges, all heads
    _, tf_peak, kind = _peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    return {"metric": "suffix_prefill_tflops_512_over_8192", "value": achieved, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 KV dequantised to fp16, fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"prefill: {T}-token chunk over {P}-token q8_0 prefix, {HQ} Q / {HKV} KV heads, d={D}, {LAYERS} layers "
                                   f"(BASELINE configs[2]); kv heads split over {world} GPU(s); kernel {args.prefill_kernel}", "l2": "L2 flushed implicitly: 16 layer caches of 19 MB rotate"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s", "frac": achieved / tf_peak,
                         "traffic": None, "peak_kind": f"{kind} (bf16_tflops_sustained)"},
            "gpu_launches": args.steps * LAYERS * (2 if ws is None else 3)}


def run_seqshard(args, torch, dist, rank, world, local_rank):
    """One 131072-token session, KV sharded by position over the ranks.  Per layer each rank reduces its shard to one
    (m, l, acc) partial per query head; with `--exchange kernel` (default) the decode kernel itself stores that
    partial into every peer's exchange buffer over NVLink and merges what it receives, with `--exchange nccl` the
    partials are all-gathered by NCCL and merged by a second kernel."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import open_exchange, shard_range

    L, HQ, HKV, D, LAYERS = args.context if args.context != 32768 else 131072, 32, 8, 128, args.layers
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
    if in_kernel and LAYERS % 2:
        raise SystemExit("seqshard --exchange kernel alternates two exchange phases per layer: use an even --layers")
    exchange = open_exchange(dist, HQ, D) if in_kernel else None
    kv.set_launch_overlap(0 if (args.no_overlap or (dist is not None and not in_kernel)) else 1)

    def step():
        for l in range(LAYERS):
            if dist is None:
                kv.launch_decode_attention_quant(views[l], q[l], query_heads=HQ, scale=D ** -0.5, cache_length=n, output=out[l], workspace=ws)
                continue
            if in_kernel:
                kv.launch_decode_attention_sharded(views[l], q[l], exchange, query_heads=HQ, scale=D ** -0.5, range_begin=0,
                                                   range_end=n, phase=l & 1, output=out[l], workspace=ws)
                continue
            kv.launch_decode_partials(views[l], q[l], query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=n,
                                      part_m=pm, part_l=pl, part_acc=pa, workspace=ws)
            dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))     # 16.6 KB per rank: the one exchange step
            kv.launch_merge_partials_packed(gathered, num_parts=world, query_heads=HQ, head_dim=D, output=out[l])

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
    checksum = float(out.double().abs().sum().item())   # identical on every rank when the exchange is right
    checksum_spread = 0.0
    if dist is not None:
        sums = [None] * world
        dist.all_gather_object(sums, checksum)
        checksum_spread = (max(sums) - min(sums)) / max(abs(max(sums)), 1e-30)
    if exchange is not None:
        dist.barrier()
        exchange.destroy()
    bw_peak, _, kind = _peaks()
    bytes_total = LAYERS * L * HKV * 136 * 2
    achieved = bytes_total / (ms * 1e-3) / 1e9
    return {"metric": "q8_0_kv_decode_tokens_per_s_128k_ctx_sequence_sharded", "value": 1000.0 / ms, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"seqshard: one {L}-token session, {LAYERS} layers, {HQ} Q / {HKV} KV heads, d={D}, q8_0; positions sharded over "
                                   f"{world} GPU(s); per layer exchange of {HQ}x({D}+2) fp32 per rank "
                                   f"({'peer stores + merge inside the decode kernel' if in_kernel else 'NCCL all-gather + merge kernel'}; BASELINE configs[4])",
                       "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak * world, "unit": "GB/s", "frac": achieved / (bw_peak * world),
                         "traffic": None, "peak_kind": f"{kind} x {world} GPUs"},
            "merge_bytes_per_layer_per_rank": HQ * (D + 2) * 4, "output_checksum": checksum, "output_checksum_spread_over_ranks": checksum_spread,
            "gpu_launches": args.steps * LAYERS * (1 if (dist is None or in_kernel) else 3)}


def run_batched(args, torch, dist, rank, world, local_rank):
    """64 sessions with context lengths uniform in [512, 16384] (seeded), one decode step each per layer in ONE launch,
    plus 16 sessions restored from a shared 4096-token prefix snapshot; sessions are bin-packed over the ranks."""
    from miinfer_b200 import kv
    from miinfer_b200.partition import partition_sessions, pick_batched_splits

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
    S = len(mine)
    g = torch.Generator(device="cuda"); g.manual_seed(rank)
    q = torch.randn(LAYERS, S, HQ, D, generator=g, device="cuda").half()
    out = torch.zeros(LAYERS, S, HQ, D, device="cuda")
    lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ws = kv.decode_workspace(HQ, D, S)
    tables = [kv.view_table(S) for _ in range(LAYERS)]
    stream = torch.cuda.current_stream()

    # restore of the snapshot sessions: device-to-device clone of the first 4096 positions, timed on its own
    def restore():
        for l in range(LAYERS):
            for j, i in enumerate(mine):
                if i >= 64:
                    caches[l][j].clone_prefix_from(proto[l], 4096)
    restore_ms = _time(torch, dist, stream, restore, 1, 3) if restored or dist is not None else 0.0
    # the host knows this step's lengths: pick the split count that fills whole waves of CTAs (0 = library default)
    splits = 0 if getattr(args, "default_splits", False) else pick_batched_splits(lengths, HKV)
    kv.set_launch_overlap(0 if args.no_overlap else 1)
    for l in range(LAYERS):   # fills the device view tables once
        kv.launch_decode_attention_batched([c.view() for c in caches[l]], tables[l], lens, max(lengths), q[l], query_heads=HQ,
                                           scale=D ** -0.5, output=out[l], workspace=ws, num_splits=splits)

    def step():
        for l in range(LAYERS):
            kv.launch_decode_attention_batched(None, tables[l], lens, max(lengths), q[l], query_heads=HQ, scale=D ** -0.5,
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
    bw_peak, _, kind = _peaks()
    bytes_total = LAYERS * sum(lengths_all) * HKV * 136 * 2
    achieved = bytes_total / (ms * 1e-3) / 1e9
    return {"metric": "batched_decode_session_steps_per_s", "value": len(lengths_all) * 1000.0 / ms, "unit": f"session-steps/s over {LAYERS} layers",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"batched: 64 sessions U[512,16384] + 16 restored from a 4096-token snapshot, {LAYERS} layers, {HQ} Q / {HKV} KV, d={D}, "
                                   f"q8_0; sessions bin-packed over {world} GPU(s) (BASELINE configs[3])", "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": bw_peak * world, "unit": "GB/s", "frac": achieved / (bw_peak * world),
                         "traffic": None, "peak_kind": f"{kind} x {world} GPUs"},
            "splits_of_longest_session": splits, "restore_ms_16_sessions": restore_ms, "restore_bytes": LAYERS * 16 * 4096 * HKV * 136 * 2, "gpu_launches": args.steps * LAYERS}


def run(args, torch, dist, rank, world, local_rank):
    fn = {"prefill": run_prefill, "seqshard": run_seqshard, "batched": run_batched}.get(args.workload)
    if fn is None:
        raise SystemExit(f"unknown workload {args.workload}")
    line = fn(args, torch, dist, rank, world, local_rank)
    return line if rank == 0 else None
