"""GPU parity: split-K GQA decode attention against the oracle's fp32-accumulated
two-pass reference, max-abs <= 2e-3 (the tolerance the path's specification states),
through the C ABI."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_attention_close, to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu
TOL = 2.0e-3


def filled(rng, L, H, d, qb, mode, cap=None, std=1.0):
    host = ko.HostCache(cap or L, H, d, qb, mode)
    host.append(ko.normal_f16(rng, (L, H * d), std).astype(np.float32), ko.normal_f16(rng, (L, H * d), std).astype(np.float32),
                None, 0, rope_mode=0)
    return host


def gpu_decode(st, q, Hq, scale, length, *, gate=None, num_splits=0, decode_state=None):
    d = st.head_dim
    out = torch.full((Hq, d), float("nan"), device="cuda")
    gated = torch.full((Hq, d), float("nan"), device="cuda")
    ws = kv.decode_workspace(Hq, d, 1)
    kv.launch_decode_attention_quant(st.view(), q, query_heads=Hq, scale=scale, cache_length=length,
                                     decode_state=decode_state, output=out, gate=gate, gated_output=gated,
                                     workspace=ws, num_splits=num_splits)
    torch.cuda.synchronize()
    return out.cpu().numpy(), gated.cpu().numpy()


# (d, H, Hq, qblock, mode, L)
SHAPES = [
    (128, 8, 32, 32, 3, 4097),     # single-layer decode step over a 4096-token context
    (128, 8, 32, 32, 3, 1),
    (128, 8, 32, 32, 3, 31),
    (128, 8, 32, 32, 3, 1025),
    (256, 4, 24, 32, 3, 777),      # hybrid-model shape, q8_0 blocks
    (256, 4, 24, 256, 3, 2049),    # the reference's row-scale format
    (256, 4, 24, 256, 1, 300),
    (256, 4, 24, 256, 2, 300),
    (256, 4, 24, 256, 0, 300),
    (128, 2, 2, 32, 3, 100),       # no GQA sharing
    (128, 1, 8, 128, 3, 515),      # group of 8
]


@pytest.mark.parametrize("d,H,Hq,qb,mode,L", SHAPES)
@pytest.mark.parametrize("path", ["auto", "mma", "generic"])
def test_decode_matches_two_pass_reference(cuda, d, H, Hq, qb, mode, L, path):
    rng = np.random.default_rng(d + L + mode)
    host = filled(rng, L, H, d, qb, mode, cap=(L + 5 + 7) // 8 * 8)
    st = upload(host)
    v = st.view()
    streaming = mode == 3 and d == 128 and Hq // H in (1, 2, 4)
    wide = mode == 3 and d == 256 and Hq // H in (4, 6, 8)
    assert kv.decode_kernel_kind(v, Hq) == (1 if streaming else 2 if wide else 0)
    q16 = ko.normal_f16(rng, (Hq, d))
    gate = rng.standard_normal((Hq, d)).astype(np.float32)
    ref, ref_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, L, gate)
    flag = kv.FORCE_GENERIC if path == "generic" else 0
    kv.set_decode_kernel(1 if path == "mma" else 0)     # which streaming kernel serves the int8 caches
    try:
        for q_dev in (to_dev(q16), to_dev(q16.astype(np.float32))):       # fp16 and fp32 queries
            out, gated = gpu_decode(st, q_dev, Hq, d ** -0.5, L, gate=to_dev(gate), num_splits=flag)
            assert_attention_close(out, ref, f"decode {path} d={d} H={H}/{Hq} qb={qb} mode={mode} L={L}")
            assert_attention_close(gated, ref_g, f"decode {path} gated")
    finally:
        kv.set_decode_kernel(0)


def test_decode_odd_capacity_uses_generic_kernel_and_still_matches(cuda):
    rng = np.random.default_rng(12)
    host = filled(rng, 700, 8, 128, 32, 3, cap=701)     # scale-plane tiles would not be 16-byte aligned
    st = upload(host)
    assert kv.decode_kernel_kind(st.view(), 32) == 0
    q16 = ko.normal_f16(rng, (32, 128))
    ref, _ = host.decode_ref(q16.astype(np.float32), 128 ** -0.5, 700)
    out, _ = gpu_decode(st, to_dev(q16), 32, 128 ** -0.5, 700)
    assert np.max(np.abs(out - ref)) <= TOL


def test_decode_split_count_invariance_and_determinism(cuda):
    rng = np.random.default_rng(77)
    host = filled(rng, 3000, 8, 128, 32, 3)
    st = upload(host)
    q = to_dev(ko.normal_f16(rng, (32, 128)))
    ref, _ = host.decode_ref(q.float().cpu().numpy(), 128 ** -0.5, 3000)
    outs = []
    for splits in (1, 2, 5, 16, 37, 64, 128):
        for flag, choice in ((0, 0), (0, 1), (kv.FORCE_GENERIC, 0)):
            kv.set_decode_kernel(choice)
            try:
                out, _ = gpu_decode(st, q, 32, 128 ** -0.5, 3000, num_splits=splits | flag)
            finally:
                kv.set_decode_kernel(0)
            assert np.max(np.abs(out - ref)) <= TOL, (splits, flag, choice)
            outs.append(out)
    # invariance up to rounding, not bit equality (the tcgen05 kernel carries the weights as 16-bit fixed point per tile)
    assert max(np.max(np.abs(o - outs[0])) for o in outs) <= 5e-5
    for choice in (0, 1):
        kv.set_decode_kernel(choice)
        try:
            a, _ = gpu_decode(st, q, 32, 128 ** -0.5, 3000)
            for _ in range(8):
                b, _ = gpu_decode(st, q, 32, 128 ** -0.5, 3000)
                assert np.array_equal(a, b)   # replay is bit-identical
        finally:
            kv.set_decode_kernel(0)


def test_decode_peaked_softmax_and_large_magnitudes(cuda):
    # one key aligned with the query dominates the softmax; values have a large range
    rng = np.random.default_rng(5)
    L, H, Hq, d = 2000, 8, 32, 128
    kf = ko.normal_f16(rng, (L, H * d)).astype(np.float32)
    vf = (ko.normal_f16(rng, (L, H * d)).astype(np.float32) * 8).astype(np.float16).astype(np.float32)
    q16 = ko.normal_f16(rng, (Hq, d), 2.0)
    for h in range(H):
        kf[1234, h * d:(h + 1) * d] = q16[h * 4].astype(np.float32) * 1.5
    host = ko.HostCache(L, H, d, 32, 3)
    host.append(kf, vf, None, 0, rope_mode=0)
    st = upload(host)
    ref, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, L)
    for flag in (0, kv.FORCE_GENERIC):
        out, _ = gpu_decode(st, to_dev(q16), Hq, d ** -0.5, L, num_splits=flag)
        assert np.max(np.abs(out - ref)) <= TOL * max(1.0, np.abs(ref).max() / 4)


def test_decode_length_from_device_state_and_quirk_free_length(cuda):
    # L = position + 1: entries 0..position, including the just-appended token
    rng = np.random.default_rng(6)
    host = filled(rng, 600, 8, 128, 32, 3, cap=1024)
    st = upload(host)
    q = to_dev(ko.normal_f16(rng, (32, 128)))
    ref, _ = host.decode_ref(q.float().cpu().numpy(), 128 ** -0.5, 600)
    state = kv.make_decode_state(599)
    for flag in (0, kv.FORCE_GENERIC):
        out, _ = gpu_decode(st, q, 32, 128 ** -0.5, 0, decode_state=state, num_splits=flag)
        assert np.max(np.abs(out - ref)) <= TOL
    # attending one slot too many (the reference's non-graph path quirk) or too few is visible
    wrong, _ = host.decode_ref(q.float().cpu().numpy(), 128 ** -0.5, 599)
    assert np.max(np.abs(wrong - ref)) > 1e-4


def test_decode_after_gpu_append_end_to_end(cuda):
    # build the whole cache through the append kernel (RoPE at true positions), then attend: config 1 shape
    rng = np.random.default_rng(8)
    L, H, Hq, d = 257, 8, 32, 128
    k16, v16 = ko.normal_f16(rng, (L, H * d)), ko.normal_f16(rng, (L, H * d))
    host = ko.HostCache(L, H, d, 32, 3)
    host.append(k16.astype(np.float32), v16.astype(np.float32), None, 0, rope_mode=1)
    st = kv.AttentionLayerKvCacheStorage(L, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=d, qblock=32)
    kv.launch_kv_store_quant(st.view(), to_dev(k16[:L - 1]), to_dev(v16[:L - 1]), None, L - 1, 0, rope_mode=kv.RopeMode.NEOX_FULL)
    kv.launch_kv_store_quant(st.view(), to_dev(k16[L - 1:]), to_dev(v16[L - 1:]), None, 1, L - 1, rope_mode=kv.RopeMode.NEOX_FULL)
    q16 = ko.normal_f16(rng, (Hq, d))
    ref, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, L)
    out, _ = gpu_decode(st, to_dev(q16), Hq, d ** -0.5, L)
    assert np.max(np.abs(out - ref)) <= TOL


def test_decode_batched_variable_lengths(cuda):
    rng = np.random.default_rng(9)
    H, Hq, d = 8, 32, 128
    lengths = [1, 37, 512, 1300, 64, 2049]
    hosts = [filled(rng, L, H, d, 32, 3, cap=(L + 7 + 7) // 8 * 8) for L in lengths]
    sts = [upload(h) for h in hosts]
    q16 = ko.normal_f16(rng, (len(lengths), Hq, d))
    table = kv.view_table(len(lengths))
    lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ws = kv.decode_workspace(Hq, d, len(lengths))
    for flag in (0, kv.FORCE_GENERIC):
        out = torch.full((len(lengths), Hq, d), float("nan"), device="cuda")
        kv.launch_decode_attention_batched([s.view() for s in sts], table, lens, max(lengths), to_dev(q16),
                                           query_heads=Hq, scale=d ** -0.5, output=out, workspace=ws, num_splits=flag)
        torch.cuda.synchronize()
        for i, h in enumerate(hosts):
            ref, _ = h.decode_ref(q16[i].astype(np.float32), d ** -0.5, lengths[i])
            assert np.max(np.abs(out[i].cpu().numpy() - ref)) <= TOL, (i, flag)
    # second call reusing the device view table
    out2 = torch.zeros_like(out)
    kv.launch_decode_attention_batched(None, table, lens, max(lengths), to_dev(q16), query_heads=Hq, scale=d ** -0.5,
                                       output=out2, workspace=ws)
    torch.cuda.synchronize()
    for i, h in enumerate(hosts):
        ref, _ = h.decode_ref(q16[i].astype(np.float32), d ** -0.5, lengths[i])
        assert np.max(np.abs(out2[i].cpu().numpy() - ref)) <= TOL, i


def test_sequence_shard_partials_merge_to_full_attention(cuda):
    rng = np.random.default_rng(10)
    L, H, Hq, d = 4096, 8, 32, 128
    host = filled(rng, L, H, d, 32, 3)
    st = upload(host)
    q16 = ko.normal_f16(rng, (Hq, d))
    ref, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, L)
    ws = kv.decode_workspace(Hq, d, 1)
    for shards in (2, 4, 8):
        pm = torch.empty(shards, Hq, device="cuda"); pl = torch.empty(shards, Hq, device="cuda")
        pa = torch.empty(shards, Hq, d, device="cuda")
        per = L // shards
        for r in range(shards):
            kv.launch_decode_partials(st.view(), to_dev(q16), query_heads=Hq, scale=d ** -0.5, range_begin=r * per,
                                      range_end=(r + 1) * per, part_m=pm[r], part_l=pl[r], part_acc=pa[r], workspace=ws)
        # device partial of shard 0 agrees with the oracle's kernel-order partial reduced the same way
        om, ol, oa = host.decode_partials(q16.astype(np.float32), d ** -0.5, 0, per, 1)
        scale_fix = np.exp(om[0] - pm[0].cpu().numpy())
        np.testing.assert_allclose(pl[0].cpu().numpy(), ol[0] * scale_fix, rtol=2e-4)
        out = torch.empty(Hq, d, device="cuda")
        kv.launch_merge_partials(pm, pl, pa, num_parts=shards, query_heads=Hq, head_dim=d, output=out)
        torch.cuda.synchronize()
        assert np.max(np.abs(out.cpu().numpy() - ref)) <= TOL
    # merge kernel alone == oracle merge on the same partials, including an empty part
    pm2 = torch.cat([pm, torch.full((1, Hq), float("-inf"), device="cuda")])
    pl2 = torch.cat([pl, torch.zeros(1, Hq, device="cuda")])
    pa2 = torch.cat([pa, torch.zeros(1, Hq, d, device="cuda")])
    out2 = torch.empty(Hq, d, device="cuda")
    kv.launch_merge_partials(pm2, pl2, pa2, num_parts=shards + 1, query_heads=Hq, head_dim=d, output=out2)
    o_ref, _ = ko.merge_partials(pm2.cpu().numpy(), pl2.cpu().numpy(), pa2.cpu().numpy())
    assert np.max(np.abs(out2.cpu().numpy() - o_ref)) <= 1e-5


def test_decode_workspace_too_small_and_bad_heads(cuda):
    st = kv.AttentionLayerKvCacheStorage(64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=8, head_dim=128, qblock=32)
    q = torch.zeros(32, 128, device="cuda", dtype=torch.float16)
    out = torch.zeros(32, 128, device="cuda")
    with pytest.raises(kv.B200KvError) as e:
        kv.launch_decode_attention_quant(st.view(), q, query_heads=32, scale=0.1, cache_length=64, output=out,
                                         workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    assert e.value.status == -5
    with pytest.raises(kv.B200KvError):
        kv.launch_decode_attention_quant(st.view(), q, query_heads=30, scale=0.1, cache_length=64, output=out,
                                         workspace=kv.decode_workspace(32, 128))


def test_decode_loop_with_launch_overlap_matches_serial(cuda):
    """A short decode loop (append + attention per layer, positions from device state) with
    programmatic launch overlap on must give the same caches and outputs as with it off,
    eagerly and under CUDA-graph replay."""
    rng = np.random.default_rng(33)
    H, Hq, d, L0, layers, steps = 8, 32, 128, 1000, 3, 5
    k0 = [to_dev(ko.normal_f16(rng, (L0, H * d))) for _ in range(layers)]
    v0 = [to_dev(ko.normal_f16(rng, (L0, H * d))) for _ in range(layers)]
    qs = to_dev(ko.normal_f16(rng, (steps, layers, Hq, d)))
    kn = to_dev(ko.normal_f16(rng, (steps, layers, 1, H * d)))
    vn = to_dev(ko.normal_f16(rng, (steps, layers, 1, H * d)))

    def run(overlap, use_graph):
        kv.set_launch_overlap(overlap)
        try:
            sts = [kv.AttentionLayerKvCacheStorage(1024, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=d, qblock=32) for _ in range(layers)]
            for l in range(layers):
                kv.launch_kv_store_quant(sts[l].view(), k0[l], v0[l], None, L0, 0, rope_mode=kv.RopeMode.NEOX_FULL)
            state = kv.make_decode_state(L0)
            ws = kv.decode_workspace(Hq, d)
            outs = torch.zeros(steps, layers, Hq, d, device="cuda")
            q_cur = torch.zeros(layers, Hq, d, device="cuda", dtype=torch.float16)
            k_cur = torch.zeros(layers, 1, H * d, device="cuda", dtype=torch.float16)
            v_cur = torch.zeros_like(k_cur)
            out_cur = torch.zeros(layers, Hq, d, device="cuda")

            def step():
                for l in range(layers):
                    kv.launch_kv_store_quant(sts[l].view(), k_cur[l], v_cur[l], None, 1, 0, rope_mode=kv.RopeMode.NEOX_FULL,
                                             decode_state=state)
                    kv.launch_decode_attention_quant(sts[l].view(), q_cur[l], query_heads=Hq, scale=d ** -0.5,
                                                     decode_state=state, output=out_cur[l], workspace=ws)
                state[1] += 1

            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                graph = None
                if use_graph:
                    q_cur.copy_(qs[0]); k_cur.copy_(kn[0]); v_cur.copy_(vn[0])
                    step(); stream.synchronize()
                    state[1] = L0
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        step()
                    state[1] = L0
                for s in range(steps):
                    q_cur.copy_(qs[s]); k_cur.copy_(kn[s]); v_cur.copy_(vn[s])
                    graph.replay() if graph is not None else step()
                    outs[s].copy_(out_cur)
            torch.cuda.synchronize()
            snap = [torch.cat([st.key_cache_q8.flatten().view(torch.uint8), st.value_cache_q8.flatten().view(torch.uint8),
                               st.key_scales.flatten().view(torch.uint8), st.value_scales.flatten().view(torch.uint8)]).cpu() for st in sts]
            return outs.cpu(), snap
        finally:
            kv.set_launch_overlap(0)

    ref_out, ref_snap = run(0, False)
    assert torch.isfinite(ref_out).all() and ref_out.abs().max() > 0
    for overlap, use_graph in ((1, False), (1, True), (0, True)):
        out, snap = run(overlap, use_graph)
        assert all(torch.equal(a, b) for a, b in zip(snap, ref_snap)), (overlap, use_graph)
        assert torch.equal(out, ref_out), (overlap, use_graph, (out - ref_out).abs().max())


@pytest.mark.parametrize("qb,norm,rope,dtype", [(32, False, 1, np.float16), (128, True, 2, np.float32), (32, True, 1, np.float32)])
def test_fused_decode_step_appends_bit_exact_and_attends(cuda, qb, norm, rope, dtype):
    """b200kv_decode_step == append + decode attention: cache rows bit-equal to the oracle, output within tolerance,
    at positions that fall first, in the middle and last in a 32-position tile, eagerly and from device state."""
    rng = np.random.default_rng(91)
    H, Hq, d, L0, cap = 8, 32, 128, 700, 1024
    k0 = ko.normal_f16(rng, (L0, H * d)).astype(np.float32); v0 = ko.normal_f16(rng, (L0, H * d)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32) if norm else None
    host = ko.HostCache(cap, H, d, qb, 3)
    host.append(k0, v0, w, 0, rope_mode=rope)
    st = upload(host)
    ws = kv.decode_workspace(Hq, d)
    state = kv.make_decode_state(0)
    wd = None if w is None else to_dev(w)
    for step, position in enumerate(range(L0, L0 + 70)):
        kn = ko.normal_f16(rng, (1, H * d)) if dtype == np.float16 else rng.standard_normal((1, H * d), dtype=np.float32)
        vn = ko.normal_f16(rng, (1, H * d)) if dtype == np.float16 else rng.standard_normal((1, H * d), dtype=np.float32)
        q16 = ko.normal_f16(rng, (Hq, d))
        host.append(kn.astype(np.float32), vn.astype(np.float32), w, position, rope_mode=rope)
        out = torch.full((Hq, d), float("nan"), device="cuda")
        if step % 2:
            state[1] = position
            kv.launch_decode_step(st.view(), to_dev(kn), to_dev(vn), to_dev(q16), query_heads=Hq, scale=d ** -0.5, decode_state=state,
                                  k_norm_weight=wd, rope_mode=kv.RopeMode(rope), output=out, workspace=ws)
        else:
            kv.launch_decode_step(st.view(), to_dev(kn), to_dev(vn), to_dev(q16), query_heads=Hq, scale=d ** -0.5, position=position,
                                  k_norm_weight=wd, rope_mode=kv.RopeMode(rope), output=out, workspace=ws)
        torch.cuda.synchronize()
        if step in (0, 1, 27, 28, 29, 60, 69):     # 700 % 32 == 28: steps 27/28/29 straddle a tile boundary
            ref, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, position + 1)
            assert np.max(np.abs(out.cpu().numpy() - ref)) <= TOL, position
    from gpu_util import assert_planes_equal
    assert_planes_equal(st, host, "after 70 fused decode steps")
    # the fallback (generic kernel) gives the same planes and outputs
    st2 = upload(host)
    kn, vn, q16 = ko.normal_f16(rng, (1, H * d)), ko.normal_f16(rng, (1, H * d)), ko.normal_f16(rng, (Hq, d))
    host.append(kn.astype(np.float32), vn.astype(np.float32), w, L0 + 70, rope_mode=rope)
    out = torch.empty(Hq, d, device="cuda")
    kv.launch_decode_step(st2.view(), to_dev(kn), to_dev(vn), to_dev(q16), query_heads=Hq, scale=d ** -0.5, position=L0 + 70,
                          k_norm_weight=wd, rope_mode=kv.RopeMode(rope), output=out, workspace=ws, num_splits=kv.FORCE_GENERIC)
    torch.cuda.synchronize()
    assert_planes_equal(st2, host, "fallback decode step")
    ref, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, L0 + 71)
    assert np.max(np.abs(out.cpu().numpy() - ref)) <= TOL


def test_fused_decode_step_long_context_many_tiles_per_pair(cuda):
    """The appended token's tile is the last of MANY tiles of its warp pair (the hand-shake between the pair's warps
    must not stall the earlier tiles), with launch overlap on and under graph replay."""
    rng = np.random.default_rng(92)
    H, Hq, d, L0, cap = 8, 32, 128, 20000, 20480
    host = ko.HostCache(cap, H, d, 32, 3)
    host.append(ko.normal_f16(rng, (L0, H * d)).astype(np.float32), ko.normal_f16(rng, (L0, H * d)).astype(np.float32), None, 0, rope_mode=1)
    st = upload(host)
    ws = kv.decode_workspace(Hq, d)
    state = kv.make_decode_state(L0)
    kn = to_dev(ko.normal_f16(rng, (1, H * d))); vn = to_dev(ko.normal_f16(rng, (1, H * d))); q = to_dev(ko.normal_f16(rng, (Hq, d)))
    out = torch.zeros(Hq, d, device="cuda")
    kv.set_launch_overlap(1)
    try:
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            kv.launch_decode_step(st.view(), kn, vn, q, query_heads=Hq, scale=d ** -0.5, decode_state=state, output=out, workspace=ws)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                kv.launch_decode_step(st.view(), kn, vn, q, query_heads=Hq, scale=d ** -0.5, decode_state=state, output=out, workspace=ws)
                state[1] += 1
            for _ in range(3):
                graph.replay()
        torch.cuda.synchronize()
    finally:
        kv.set_launch_overlap(0)
    kf, vf = kn.float().cpu().numpy(), vn.float().cpu().numpy()
    for pos in (L0, L0 + 1, L0 + 2):      # the eager call wrote L0, the replays L0, L0+1, L0+2
        host.append(kf, vf, None, pos, rope_mode=1)
    from gpu_util import assert_planes_equal
    assert_planes_equal(st, host, "graph-replayed fused steps")
    ref, _ = host.decode_ref(q.float().cpu().numpy(), d ** -0.5, L0 + 3)
    assert np.max(np.abs(out.cpu().numpy() - ref)) <= TOL


# (H, Hq, qblock, L): head_dim 256 on the tcgen05 stage-1 kernel
WIDE = [
    (4, 24, 32, 8200),      # the reference's geometry, q8_0 blocks, many tiles per CTA
    (4, 24, 256, 4099),     # ... with its one-scale-per-row format
    (2, 16, 32, 3001),      # 8 query heads per kv head
    (4, 16, 256, 1500),     # 4 query heads per kv head
    (4, 24, 32, 129),       # two tiles, the second one position long
]


@pytest.mark.parametrize("H,Hq,qb,L", WIDE)
def test_decode_head_dim_256_tcgen05_stage1(cuda, H, Hq, qb, L):
    d = 256
    rng = np.random.default_rng(L + Hq)
    host = filled(rng, L, H, d, qb, 3, cap=(L + 64 + 7) // 8 * 8)
    st = upload(host)
    assert kv.decode_kernel_kind(st.view(), Hq) == 2
    q16 = ko.normal_f16(rng, (Hq, d))
    gate = rng.standard_normal((Hq, d)).astype(np.float32)
    ref, ref_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, L, gate)
    generic, _ = gpu_decode(st, to_dev(q16), Hq, d ** -0.5, L, gate=to_dev(gate), num_splits=kv.FORCE_GENERIC)
    for splits in (0, 1, 3, 37):
        for q_dev in (to_dev(q16), to_dev(q16.astype(np.float32))):
            out, gated = gpu_decode(st, q_dev, Hq, d ** -0.5, L, gate=to_dev(gate), num_splits=splits)
            assert_attention_close(out, ref, f"decode d=256 tcgen05 H={H}/{Hq} qb={qb} L={L} splits={splits}")
            assert_attention_close(gated, ref_g, "decode d=256 tcgen05 gated")
            assert np.linalg.norm(out - generic) <= 5e-4 * np.linalg.norm(generic)   # same sums, 16-bit fixed-point weights per tile
    # the length from a device-side state, and replay determinism
    state = kv.make_decode_state(L - 1)
    a, _ = gpu_decode(st, to_dev(q16), Hq, d ** -0.5, 0, decode_state=state)
    assert_attention_close(a, ref, "decode d=256 tcgen05, device-side length")
    b, _ = gpu_decode(st, to_dev(q16), Hq, d ** -0.5, 0, decode_state=state)
    assert np.array_equal(a, b)


def test_decode_steps_head_dim_256_back_to_back_with_launch_overlap(cuda):
    """At head_dim 256 a decode step is the store kernel, the tcgen05 stage 1 and the merge kernel.  With launch overlap on,
    each becomes resident while its predecessor still runs (stage 1 even fetches the old cache rows) and orders itself by
    its own dependency wait: eight steps launched back to back must give, bit for bit, what the serialised launches give."""
    d, H, Hq, L0, steps = 256, 4, 24, 4000, 8
    rng = np.random.default_rng(256)
    host = filled(rng, L0, H, d, 32, 3, cap=L0 + 64)
    kn = [to_dev(ko.normal_f16(rng, (1, H * d))) for _ in range(steps)]
    vn = [to_dev(ko.normal_f16(rng, (1, H * d))) for _ in range(steps)]
    qs = [to_dev(ko.normal_f16(rng, (Hq, d))) for _ in range(steps)]
    w = to_dev((1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    results = {}
    for overlap in (0, 1):
        st = upload(host)
        ws = kv.decode_workspace(Hq, d)
        outs = torch.full((steps, Hq, d), float("nan"), device="cuda")
        kv.set_launch_overlap(overlap)
        try:
            for i in range(steps):   # host-side positions: no kernel in between that would serialise the chain
                kv.launch_decode_step(st.view(), kn[i], vn[i], qs[i], query_heads=Hq, scale=d ** -0.5, position=L0 + i,
                                      k_norm_weight=w, rope_mode=kv.RopeMode.SECTIONED64, output=outs[i], workspace=ws)
            torch.cuda.synchronize()
        finally:
            kv.set_launch_overlap(0)
        results[overlap] = (outs.cpu(), st.key_cache_q8[:, :L0 + steps].cpu(), st.value_cache_q8[:, :L0 + steps].cpu())
    assert torch.isfinite(results[1][0]).all()
    for a, b in zip(results[0], results[1]):
        assert torch.equal(a, b)
