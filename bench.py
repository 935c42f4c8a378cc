#!/usr/bin/env python
"""Benchmark of the quantized-KV decode path: q8_0-KV decode attention throughput at 32K context.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `decode32k`: a 36-layer Qwen3-8B-shaped KV decode sweep at 32K
context (32 Q / 8 KV heads, d=128, q8_0 K/V, batch 1): per layer one fused
append (fp16 K/V, NeoX RoPE) and one split-K GQA decode attention.  One "step"
is one decode step over all 36 layers; `value` is decode tokens/s with the
caches resident in HBM.  With N GPUs every rank decodes its own session (weak
scaling, no data-path collective).  Other workloads:
`seqshard` (one 128K-token session sharded by sequence over the ranks; the per-rank
partials are exchanged and merged inside the decode kernel, or by NCCL with --exchange nccl), `batched` (64 sessions of mixed
length), `prefill` (512-token suffix over an 8K prefix, d=256), `decode256` (decode attention on the reference's own 24 Q / 4 KV, d=256 geometry), `append` (the store kernel alone: 8192-token chunks at d=128,
or with --append-shape chunk256 the 512-token d=256 chunk).

The default run also measures, as sub-records of the same JSON line, the suffix-prefill
workload (`prefill`), on one GPU the head_dim-256 decode and the append workloads (`decode256`, `append`) and -- with N > 1
GPUs -- the sharded workloads (`seqshard`, `batched`)
together with their own 1-GPU times; `--no-extras` leaves them out.  After the timed region the
output of one layer is compared with the CPU oracle on the cache as it then lies (`check`),
and the step graph is replayed for two seconds with the SM clock sampled (`sustained`).

The `--impl reference` arm times the CPU restatement of the reference path
(oracle/) on the host cores; the reference itself has no CPU implementation of
the quantized path and its GPU code is HIP for gfx906 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

LAYERS, HQ, HKV, D, QB = 36, 32, 8, 128, 32
ROW = D + 2 * (D // QB)  # 136 bytes per head-row
THETA = 1.0e6

# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch at 32K context, from ncu captures of the
# two streaming kernels on a 2-layer run of the same launch size: the tcgen05 kernel 71.90 MB read + 1.46 MB written,
# the warp-level mma kernel 71.61 MB + 1.74 MB
NCU_TRAFFIC_BYTES_32K = {"tcgen05": 73_355_264, "mma": 73_352_704}


def measured_peak_gbs() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU during the timed region: through NVML (read-only queries
    from a thread, every 5 ms, so that a region of a few tens of milliseconds still gets samples), with nvidia-smi as
    the fallback where the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.proc = None
        self.thread = None
        self.sm, self.mx, self.reasons = [], 0.0, set()
        try:
            import threading

            import pynvml

            pynvml.nvmlInit()
            handle = None
            try:   # the CUDA ordinal is not NVML's index when CUDA_VISIBLE_DEVICES reorders: go by UUID
                import torch

                uuid = str(torch.cuda.get_device_properties(index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self._halt = threading.Event()

            def loop():
                while not self._halt.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        bits = int(reasons_fn(handle))
                        for bit, name in self.REASON_BITS.items():
                            if bits & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    self._halt.wait(0.005)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.thread is not None:
            self._halt.set()
            self.thread.join(timeout=2)
            sm = sorted(self.sm)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.mx or None, "reasons": sorted(self.reasons),
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=5)
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


# ---------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port on host cores
# ---------------------------------------------------------------------------------

def cpu_decode_sample(context: int, sample_layers: int, threads: int, repeats: int = 1) -> dict:
    """Times `sample_layers` layers of one decode step (append + split-K attention) of the
    oracle on `threads` host threads; returns tokens/s scaled to LAYERS layers."""
    import numpy as np

    import kvoracle as ko

    ko.set_threads(threads)
    rng = np.random.default_rng(42)
    host = ko.HostCache(context + 8, HKV, D, QB, 3)
    chunk = 4096
    for base in range(0, context - 1, chunk):
        n = min(chunk, context - 1 - base)
        host.append(ko.normal_f16(rng, (n, HKV * D)).astype(np.float32), ko.normal_f16(rng, (n, HKV * D)).astype(np.float32),
                    None, base, rope_mode=0)
    q = ko.normal_f16(rng, (HQ, D)).astype(np.float32)
    k_new = ko.normal_f16(rng, (1, HKV * D)).astype(np.float32)
    v_new = ko.normal_f16(rng, (1, HKV * D)).astype(np.float32)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for _layer in range(sample_layers):   # the same cache stands in for each sampled layer (32K x 2176 B = 71 MB >> host L2)
            host.append(k_new, v_new, None, context - 1, rope_mode=1, theta=THETA)
            host.decode_splitk(q, D ** -0.5, context, 0)
        best = min(best, time.perf_counter() - t0)
    per_token = best * LAYERS / sample_layers
    return {"value": 1.0 / per_token, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of {LAYERS} layers of one decode step at {context} context "
                      f"(append + split-K attention, oracle/kv_oracle.c), scaled x{LAYERS}/{sample_layers}",
            "seconds": best}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    ctx = 32768
    times = []
    for _ in range(args.warmup):
        cpu_decode_sample(ctx, 1, threads)
    t_all = time.perf_counter()
    res = None
    for _ in range(args.steps):
        res = cpu_decode_sample(ctx, 2, threads)
        times.append(res["seconds"] * LAYERS / 2)
    ms = 1000.0 * sum(times) / len(times)
    value = 1000.0 / ms
    line = {
        "impl": "reference", "metric": "q8_0_kv_decode_tokens_per_s_32k_ctx", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
        "config": workload_config("decode32k", ctx, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": res["sample"]},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's HIP kernels (oracle/); the reference has no CPU implementation of "
                "the quantized path and its GPU code is gfx906-only HIP",
        "wall_s": time.perf_counter() - t_all,
    }
    emit_line(line)


def workload_config(name: str, context: int, n_gpus: int) -> dict:
    return {"workload": f"{name}: {LAYERS}-layer Qwen3-8B-shaped KV decode step at {context} context: "
                        f"per layer fused append + split-K GQA attention, {HQ} Q / {HKV} KV heads, d={D}, q8_0 K/V "
                        f"(32 int8 + fp16 scale), batch 1 per GPU",
            "context": context, "layers": LAYERS, "sessions_per_gpu": 1, "parallelism": f"session-parallel x{n_gpus}",
            "l2": "inputs larger than L2: 2.57 GB of KV per step vs 126 MB L2"}


# ---------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------

def fill_cache(kv, torch, storage, tokens: int, seed: int) -> None:
    """Existing context: fp16 N(0,1) source rows quantised by the append kernel (no RoPE on filler rows)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    chunk = 8192
    width = storage.kv_heads * storage.head_dim
    for base in range(0, tokens, chunk):
        n = min(chunk, tokens - base)
        k = torch.randn(n, width, generator=g, device="cuda", dtype=torch.float32).half()
        v = torch.randn(n, width, generator=g, device="cuda", dtype=torch.float32).half()
        kv.launch_kv_store_quant(storage.view(), k, v, None, n, base, rope_mode=kv.RopeMode.NONE)


def run_decode32k(args, torch, dist, rank, world, local_rank):
    from miinfer_b200 import kv

    ctx = args.context
    cap = (ctx + args.warmup + 2 * args.steps + 256 + 63) // 64 * 64
    dev = torch.device("cuda", local_rank)
    caches = [kv.AttentionLayerKvCacheStorage(cap, kv.KvCacheQuantMode.kQ8Q8, kv_heads=HKV, head_dim=D, qblock=QB, device=dev)
              for _ in range(LAYERS)]
    for i, c in enumerate(caches):
        fill_cache(kv, torch, c, ctx - 1, seed=1000 * rank + i)
    views = [c.view() for c in caches]
    g = torch.Generator(device="cuda")
    g.manual_seed(4242 + rank)
    # a layer's inputs lie side by side, [q | new K row | new V row], so that the end-to-end path moves them with one copy
    packed = torch.randn(LAYERS, HQ * D + 2 * HKV * D, generator=g, device=dev).half()
    q = packed[:, :HQ * D].view(LAYERS, HQ, D)
    k_new = packed[:, HQ * D:HQ * D + HKV * D].view(LAYERS, 1, HKV * D)
    v_new = packed[:, HQ * D + HKV * D:].view(LAYERS, 1, HKV * D)
    out = torch.zeros(LAYERS, HQ, D, device=dev)
    ws = kv.decode_workspace(HQ, D, 1, device=dev)
    state = kv.make_decode_state(ctx - 1, device=dev)   # position of the token being appended; length = position + 1
    scale = D ** -0.5

    def layer_pass(first=0, last=LAYERS):
        for l in range(first, last):
            if args.two_launches:   # the reference's call pair: store kernel, then decode attention
                kv.launch_kv_store_quant(views[l], k_new[l], v_new[l], None, 1, 0, rope_mode=kv.RopeMode.NEOX_FULL,
                                         theta=THETA, decode_state=state)
                kv.launch_decode_attention_quant(views[l], q[l], query_heads=HQ, scale=scale, decode_state=state,
                                                 output=out[l], workspace=ws)
            else:                   # the same work as one launch (append fused into the streaming kernel)
                kv.launch_decode_step(views[l], k_new[l], v_new[l], q[l], query_heads=HQ, scale=scale, decode_state=state,
                                      rope_mode=kv.RopeMode.NEOX_FULL, theta=THETA, output=out[l], workspace=ws)

    attn_state = kv.make_decode_state(ctx - 2, device=dev)   # attention alone scans the rows that are there: position + 1 of them

    def attention_only_pass():
        for l in range(LAYERS):
            kv.launch_decode_attention_quant(views[l], q[l], query_heads=HQ, scale=scale, decode_state=attn_state,
                                             output=out[l], workspace=ws)

    # consecutive layers' kernels may overlap their ramp-up and tail (programmatic dependent launch);
    # one trailing cache row -- the token appended by the preceding kernel -- is guarded
    kv.set_launch_overlap(0 if args.no_overlap else 1)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        layer_pass()                       # eager once (loads modules) before capture
        stream.synchronize()
        state[1] = ctx - 1
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            layer_pass()
            state[1] += 1                  # device-side advance so the replay appends at the next position
        attn_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(attn_graph, stream=stream):
            attention_only_pass()
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput -------------------------------------------------
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
    barrier()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop()

    # ---- dominant kernel: decode attention alone (one launch per layer), for the roofline -----
    with torch.cuda.stream(stream):
        attn_state[1] = state[1] - 1       # the rows appended so far
        for _ in range(3):
            attn_graph.replay()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(args.steps):
            attn_graph.replay()
        a1.record(stream)
    torch.cuda.synchronize()
    length_now = int(attn_state[1].item()) + 1   # context length the attention-only replays scanned
    attn_us = 1000.0 * a0.elapsed_time(a1) / (args.steps * LAYERS)
    attn_bytes = length_now * HKV * ROW * 2 + HQ * D * 2 + HQ * D * 4

    # ---- end to end through the public API with host buffers --------------------------------
    # Every step moves all 36 layers' inputs from pinned host memory (they lie side by side) and all 36 outputs back; the
    # copies are nodes of the step's graph, and the host waits for the whole step before the next one.  The inputs travel
    # as two copies -- the first layers' on the step's own stream, the rest on a side stream while those layers run -- and
    # so do the outputs: all but the last layers' leave on the side stream while the last layers run.  (One copy each
    # way, nothing overlapped: 0.69 ms.  A copy per layer and direction: 0.84 ms -- 72 small copy nodes and their
    # edges cost more than they hide.)
    h_in = torch.randn(LAYERS, HQ * D + 2 * HKV * D).half().pin_memory()
    h_out = torch.empty(LAYERS, HQ, D).pin_memory()
    e2e_steps = max(3, min(args.steps, 50))
    head, tail = (min(args.e2e_head, LAYERS - 1), max(LAYERS - args.e2e_tail, 1)) if LAYERS >= 3 and not args.e2e_single_copies else (LAYERS, LAYERS)
    e2e_graph, e2e_mode = None, ("one graph per step: inputs in two copies (layers 0-%d, then the rest beside them), 36 layers, outputs in two "
                                 "copies (layers 0-%d beside the last layers, then the rest)" % (head - 1, tail - 1))
    if head >= LAYERS:
        e2e_mode = "one graph per step: copy in, 36 layers, copy out"
    try:
        e2e_graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            with torch.cuda.graph(e2e_graph, stream=stream):
                if head < LAYERS:
                    side.wait_stream(stream)
                    packed[:head].copy_(h_in[:head], non_blocking=True)
                    with torch.cuda.stream(side):
                        packed[head:].copy_(h_in[head:], non_blocking=True)
                    layer_pass(0, head)
                    stream.wait_stream(side)
                    layer_pass(head, tail)
                    side.wait_stream(stream)
                    with torch.cuda.stream(side):
                        h_out[:tail].copy_(out[:tail], non_blocking=True)
                    layer_pass(tail, LAYERS)
                    h_out[tail:].copy_(out[tail:], non_blocking=True)
                    stream.wait_stream(side)
                else:
                    packed.copy_(h_in, non_blocking=True)
                    layer_pass()
                    h_out.copy_(out, non_blocking=True)
                state[1] += 1
        torch.cuda.synchronize()
    except Exception as exc:   # a driver that cannot capture the copies: the plain sequence below
        print(f"bench: end-to-end graph not captured ({exc}); copies issued around the step graph", file=sys.stderr)
        e2e_graph = None
        torch.cuda.synchronize()
    if e2e_graph is None:
        e2e_mode = "copy in, step graph, copy out, issued one after the other"
    with torch.cuda.stream(stream):
        for i in range(3 + e2e_steps):
            if i == 3:
                stream.synchronize()
                t0 = torch.cuda.Event(enable_timing=True)
                t1 = torch.cuda.Event(enable_timing=True)
                t0.record(stream)
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                packed.copy_(h_in, non_blocking=True)
                graph.replay()
                h_out.copy_(out, non_blocking=True)
            stream.synchronize()           # the caller needs the step's result before the next token
        t1.record(stream)
    barrier()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps

    # ---- the same step graph replayed for two seconds, SM clock sampled over the window --------------------
    sustained = None
    if not args.no_sustained:
        chunk = max(1, min(args.steps + args.warmup, 64))      # replays between rewinds of the position (the cache has room for these)
        first_position = ctx - 1
        s_sampler = ClockSampler(local_rank)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        replays = 0
        t_wall = time.perf_counter()
        with torch.cuda.stream(stream):
            s0.record(stream)
            while time.perf_counter() - t_wall < 2.0:
                state[1] = first_position                      # rewind: the same rows are rewritten with the same bits
                for _ in range(chunk):
                    graph.replay()
                replays += chunk
                stream.synchronize()
            s1.record(stream)
        torch.cuda.synchronize()
        s_clocks = s_sampler.stop()
        s_ms = s0.elapsed_time(s1) / replays
        sustained = {"seconds": s0.elapsed_time(s1) / 1000.0, "steps": replays, "ms_per_step": s_ms, "tokens_per_s": 1000.0 / s_ms,
                     "sm_mhz_median": s_clocks.get("sm_mhz"), "sm_max_mhz": s_clocks.get("sm_max_mhz"), "clock_samples": s_clocks.get("samples"),
                     "reasons": s_clocks.get("reasons"),
                     "ms_times_median_mhz": None if s_clocks.get("sm_mhz") is None else s_ms * s_clocks["sm_mhz"],
                     "note": "includes one host synchronisation and one position rewind per %d replays" % chunk}

    # ---- the output against the CPU oracle, on the cache as it now lies on the device (layer 0) ----------------
    check = None
    if rank == 0 and not args.no_check:
        from miinfer_b200 import workloads as wl

        ko = wl._oracle()
        ko.set_threads(os.cpu_count() or 1)
        with torch.cuda.stream(stream):
            attn_state[1] = state[1] - 1
            kv.launch_decode_attention_quant(views[0], q[0], query_heads=HQ, scale=scale, decode_state=attn_state, output=out[0], workspace=ws)
        torch.cuda.synchronize()
        rows = int(attn_state[1].item()) + 1
        host = wl.host_cache_from_planes(ko, wl.planes_of(torch, caches[0], rows), rows, HKV, D)
        ref, _ = host.decode_ref(q[0].float().cpu().numpy(), scale, rows)
        check = wl.error_record(out[0].cpu().numpy(), ref, layer=0, context=rows,
                                rows_appended_by_the_fused_step=rows - (ctx - 1))

    ms = torch.tensor([ms_total / args.steps, e2e_ms, attn_us], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms, attn_us = (float(x) for x in ms.tolist())
    if rank != 0:
        return None
    peak, peak_kind = measured_peak_gbs()
    achieved = attn_bytes / (attn_us * 1e-6) / 1e9
    step_bytes = LAYERS * (attn_bytes + HKV * D * 2 * 2 + HKV * ROW * 2)
    line = {
        "metric": "q8_0_kv_decode_tokens_per_s_32k_ctx", "value": world * 1000.0 / ms_step, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 KV / fp32 accumulate", "data": "synthetic",
        "config": workload_config("decode32k", ctx, world),
        "hbm_gbs_whole_step": step_bytes / (ms_step * 1e-3) / 1e9,
        "hbm_frac_whole_step": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_32K[args.decode_kernel] if ctx == 32768 else None, "peak_kind": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs, burst copy)",
                     "kernel": ("decode_q8_kernel (split-K stage 1 on warp-level mma, merge fused in)" if args.decode_kernel == "mma" else
                                "decode_tc5_kernel (split-K stage 1 on tcgen05 int8 MMA from TMA tiles, merge fused in)"), "us_per_launch": attn_us,
                     "algorithmic_bytes_per_launch": attn_bytes, "frac_of_nominal_8TBs": achieved / 8000.0},
        "e2e": {"value": world * 1000.0 / e2e_ms, "unit": "tokens/s",
                "h2d_bytes_per_step": int(h_in.numel() * 2),
                "d2h_bytes_per_step": int(h_out.numel() * 4), "ms_per_step": e2e_ms, "how": e2e_mode},
        "gpu_launches": args.steps * LAYERS * (2 if args.two_launches else 1),   # per layer: fused append+attention+merge
        "clocks": clocks, "check": check, "sustained": sustained,
    }
    del caches, views
    return line


_RESULT_FD = None


def keep_stdout_for_the_result() -> None:
    """Everything libraries print to standard output (NCCL's version banner, for one) is sent to standard error, so
    that standard output carries the one JSON line and nothing else."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit_line(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, text)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode32k")
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of one layer's output with the CPU oracle")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second replay window")
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-records (prefill; with N > 1 also seqshard and batched)")
    ap.add_argument("--seq-context", type=int, default=131072, help="seqshard workload: context length of the one session")
    ap.add_argument("--two-launches", action="store_true", help="append and attention as two launches per layer (A/B of the fused step)")
    ap.add_argument("--prefill-kernel", default="tcgen05", choices=["tcgen05", "mma"], help="prefill workload: which attention kernel")
    ap.add_argument("--e2e-head", type=int, default=4, help="end-to-end leg: layers whose inputs travel in the first copy")
    ap.add_argument("--e2e-tail", type=int, default=3, help="end-to-end leg: layers whose outputs travel in the last copy")
    ap.add_argument("--e2e-single-copies", action="store_true", help="end-to-end leg: one copy in and one copy out per step, nothing overlapped (A/B)")
    ap.add_argument("--no-prepare-ahead", action="store_true", help="prefill workload: every layer converts its whole prefix itself (A/B)")
    ap.add_argument("--no-overlap", action="store_true", help="launch every kernel fully serialised (A/B of launch overlap)")
    ap.add_argument("--default-splits", action="store_true", help="batched workload: leave the split count to the library (A/B of the host-side picker)")
    ap.add_argument("--exchange", default="kernel", choices=["kernel", "nccl", "nccl-c"],
                    help="seqshard workload at N>1: cross-GPU merge inside the decode kernel (peer stores) or NCCL all-gather + merge kernel")
    ap.add_argument("--decode-kernel", default="tcgen05", choices=["tcgen05", "mma"],
                    help="which streaming decode kernel serves the int8 caches (A/B): tcgen05 (default) or warp-level mma")
    ap.add_argument("--append-tokens", type=int, default=8192, help="append workload: rows per layer and launch")
    ap.add_argument("--append-shape", default="fill128", choices=["fill128", "chunk256"], help="append workload: 8 kv heads d=128 or the 512-token d=256 chunk")
    ap.add_argument("--layers", type=int, default=36, help="layers per step (36 = the benchmark; fewer only for ncu captures)")
    args = ap.parse_args()
    keep_stdout_for_the_result()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    global LAYERS
    LAYERS = args.layers

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the KV path has no CPU fallback")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    from miinfer_b200 import kv as _kv

    _kv.set_decode_kernel({"tcgen05": 0, "mma": 1}[args.decode_kernel])
    args.cpu_threads = os.cpu_count() or 1
    from miinfer_b200 import workloads

    if args.workload == "decode32k":
        line = run_decode32k(args, torch, dist, rank, world, local_rank)
        if not args.no_extras and args.layers == 36:
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            sub = workloads.extras(args, torch, dist, rank, world, local_rank)
            if rank == 0 and line is not None:
                line.update(sub)
    else:
        line = workloads.run(args, torch, dist, rank, world, local_rank)
    if rank == 0 and line is not None:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cpu = cpu_decode_sample(args.context, 2, threads)
            cpu.pop("seconds", None)
            line["cpu_baseline"] = cpu
        emit_line(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
