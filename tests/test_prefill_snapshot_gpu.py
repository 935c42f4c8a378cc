"""GPU parity: suffix/prefill attention over a quantized prefix, and prefix
snapshot/restore, against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_planes_equal, device_storage_like, to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu
TOL = 2.0e-3


def filled(rng, L, H, d, qb, mode, cap=None, std=1.0):
    host = ko.HostCache(cap or L, H, d, qb, mode)
    host.append(ko.normal_f16(rng, (L, H * d), std).astype(np.float32), ko.normal_f16(rng, (L, H * d), std).astype(np.float32),
                None, 0, rope_mode=0)
    return host


# (prefix, suffix, d, H, Hq, qb, mode)
SUFFIX = [
    (64, 16, 256, 4, 24, 256, 3),     # the reference's own test ladder, tests/qwen3_quant_kv_attention_test.cpp:82-87
    (512, 64, 256, 4, 24, 256, 3),
    (512, 64, 256, 4, 24, 32, 3),     # same with q8_0 blocks (the suffix-prefill workload's format)
    (100, 33, 256, 4, 24, 256, 1),
    (100, 33, 256, 4, 24, 256, 2),
    (0, 40, 256, 4, 24, 32, 3),       # cold prefill: no prefix at all
    (300, 17, 128, 8, 32, 32, 3),
]


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("P,T,d,H,Hq,qb,mode", SUFFIX)
def test_suffix_attention_matches_reference(cuda, P, T, d, H, Hq, qb, mode, kernel):
    rng = np.random.default_rng(P + T + mode)
    host = filled(rng, P + T, H, d, qb, mode, cap=P + T + 128, std=0.5)   # N(0, 0.5) as the reference's test
    st = upload(host)
    q = (rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)
    gate = (rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)
    ref = host.suffix_ref(q, gate, P, d ** -0.5)
    out = torch.full((T, Hq, d), float("nan"), device="cuda")
    # with the fp16 scratch the tcgen05 kernel runs; without a workspace the register-resident mma.sync kernel
    ws = kv.prefill_workspace(host.capacity, H, d) if kernel == "tcgen05" else None
    kv.launch_suffix_attention_quant(st.view(), to_dev(q), to_dev(gate), out, ws, T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.max(np.abs(got - ref)) <= TOL
    # the reference's own gate for this path: cosine >= 0.999, MAE <= 0.05 (test :278)
    cos = float((got * ref).sum() / (np.linalg.norm(got) * np.linalg.norm(ref) + 1e-12))
    assert cos >= 0.999 and np.mean(np.abs(got - ref)) <= 0.05
    # ungated + fp16 queries + device-side prefill state
    q16 = q.astype(np.float16)
    ref2 = host.suffix_ref(q16.astype(np.float32), None, P, d ** -0.5)
    out2 = torch.empty((T, Hq, d), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), to_dev(q16), None, out2, ws, T, 0, query_heads=Hq, scale=d ** -0.5,
                                     prefill_state=kv.make_prefill_state(P, T))
    torch.cuda.synchronize()
    assert np.max(np.abs(out2.cpu().numpy() - ref2)) <= TOL


def test_suffix_is_causal_inside_the_chunk(cuda):
    # changing a later chunk position must not change an earlier token's output
    rng = np.random.default_rng(3)
    P, T, d, H, Hq = 50, 12, 256, 4, 24
    host = filled(rng, P + T, H, d, 32, 3)
    st = upload(host)
    q = to_dev(ko.normal_f16(rng, (T, Hq, d)))
    ws = kv.prefill_workspace(P + T, H, d)
    a = torch.empty((T, Hq, d), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), q, None, a, ws, T, P, query_heads=Hq, scale=d ** -0.5)
    st.value_cache_q8[:, P + 6:] = 77
    b = torch.empty((T, Hq, d), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), q, None, b, ws, T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    assert torch.equal(a[:6], b[:6]) and not torch.equal(a[6:], b[6:])


@pytest.mark.parametrize("mode,qb,d,H", [(3, 32, 128, 8), (3, 256, 256, 4), (1, 256, 256, 4), (2, 32, 256, 4), (0, 128, 128, 8)])
def test_snapshot_save_restore_matches_reference_layout(cuda, mode, qb, d, H):
    rng = np.random.default_rng(17 + mode)
    cap, tokens = 97, 41
    host = filled(rng, cap, H, d, qb, mode)
    st = upload(host)
    blob_ref = host.download_raw(tokens)
    assert st.raw_tokens_bytes(tokens) == blob_ref.size
    # save to pageable host, pinned host and device memory: identical bytes, identical to the oracle's layout
    for dst in (torch.zeros(blob_ref.size, dtype=torch.uint8), torch.zeros(blob_ref.size, dtype=torch.uint8).pin_memory(),
                torch.zeros(blob_ref.size, dtype=torch.uint8, device="cuda")):
        st.download_raw(dst, tokens)
        torch.cuda.synchronize()
        assert np.array_equal(dst.cpu().numpy(), blob_ref)
    # restore into a cache of another capacity: first `tokens` rows equal, the rest untouched (zero)
    other_host = ko.HostCache(cap + 30, H, d, qb, mode)
    other_host.upload_raw(blob_ref, tokens)
    other = device_storage_like(other_host)
    other.upload_raw(torch.from_numpy(blob_ref).pin_memory(), tokens)
    torch.cuda.synchronize()
    assert_planes_equal(other, other_host, "restore")
    # device-to-device clone gives the same planes
    third = device_storage_like(other_host)
    third.clone_prefix_from(st, tokens)
    torch.cuda.synchronize()
    assert_planes_equal(third, other_host, "clone")
    with pytest.raises(RuntimeError):
        st.download_raw(torch.zeros(10, dtype=torch.uint8), cap + 1)     # the reference throws (kv_cache.cpp:228-230)


def test_restored_session_decodes_like_the_original(cuda):
    # cold vs restored outputs must be identical (the reference's persistent-session gate)
    rng = np.random.default_rng(23)
    H, Hq, d, P = 8, 32, 128, 4096
    host = filled(rng, P, H, d, 32, 3, cap=P + 8)
    st = upload(host)
    blob = torch.zeros(st.raw_tokens_bytes(P), dtype=torch.uint8, device="cuda")
    st.download_raw(blob, P)
    restored = device_storage_like(host)
    restored.upload_raw(blob, P)
    q = to_dev(ko.normal_f16(rng, (Hq, d)))
    ws = kv.decode_workspace(Hq, d)
    outs = []
    for s in (st, restored):
        o = torch.empty(Hq, d, device="cuda")
        kv.launch_decode_attention_quant(s.view(), q, query_heads=Hq, scale=d ** -0.5, cache_length=P, output=o, workspace=ws)
        outs.append(o)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_native_cache_object_lifecycle(cuda):
    import ctypes as C
    from miinfer_b200._lib import View, lib

    handle = C.c_void_p()
    assert lib.b200kv_cache_create(C.byref(handle), 33, 8, 128, 32, 3) == 0
    v = View()
    assert lib.b200kv_cache_view(handle, C.byref(v)) == 0
    assert v.capacity == 33 and v.key_q8 and v.key_scales and not v.key_f16
    x = torch.randn(3, 1024, device="cuda", dtype=torch.float16)
    assert lib.b200kv_append(C.byref(v), x.data_ptr(), x.data_ptr(), 0, None, 1, 1e6, 1e-6, 3, 4, None, None, None) == 0
    blob = torch.zeros(lib.b200kv_snapshot_bytes(C.byref(v), 8), dtype=torch.uint8, device="cuda")
    assert lib.b200kv_snapshot_save(C.byref(v), 8, blob.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert blob.count_nonzero().item() > 0
    assert lib.b200kv_cache_reset(handle, None) == 0
    assert lib.b200kv_snapshot_save(C.byref(v), 8, blob.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert blob.count_nonzero().item() == 0
    assert lib.b200kv_cache_destroy(handle) == 0


def test_suffix_tcgen05_many_tiles_rescale_and_ragged_rows(cuda):
    """Long prefix (many KV tiles, both ring stages reused many times), a query whose score maximum keeps growing
    (exercises the lazy O rescale in TMEM), and a row count that is not a multiple of 128."""
    rng = np.random.default_rng(77)
    P, T, d, H, Hq = 3000, 70, 256, 4, 24
    kf = ko.normal_f16(rng, (P + T, H * d), 0.5).astype(np.float32)
    vf = ko.normal_f16(rng, (P + T, H * d), 1.0).astype(np.float32)
    q = (rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)
    # keys aligned with token 3's query of head 0, growing along the sequence: the running maximum jumps by > 2^8 repeatedly
    for i, pos in enumerate(range(100, P, 400)):
        kf[pos, :d] = q[3, 0] * (0.8 + 0.45 * i)
    host = ko.HostCache(P + T, H, d, 32, 3)
    host.append(kf, vf, None, 0, rope_mode=0)
    st = upload(host)
    ref = host.suffix_ref(q, None, P, d ** -0.5)
    out = torch.full((T, Hq, d), float("nan"), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), to_dev(q), None, out, kv.prefill_workspace(P + T, H, d), T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) <= TOL * max(1.0, float(np.abs(ref).max()))


def test_session_file_save_find_load_gives_identical_decode(cuda, tmp_path):
    """Cold vs restored-from-disk must decode identically (the reference's persistent-session gate,
    bench/v2_0028_persistent_session_bench.cpp:235-257), and a file for another quant mode must be refused."""
    rng = np.random.default_rng(29)
    H, Hq, d, P, layers = 8, 32, 128, 600, 3
    hosts = [filled(rng, P, H, d, 32, 3, cap=640) for _ in range(layers)]
    sts = [upload(h) for h in hosts]
    tokens = [int(t) for t in rng.integers(0, 150000, P)]
    name = f"sess_{kv.token_sequence_hash(tokens):016x}_p{P}.miinfer"
    kv.save_session(str(tmp_path / name), "qwen3-8b", "q4_0", tokens, sts)
    prompt = tokens + [11, 12, 13]
    found = kv.find_matching_session(str(tmp_path), "qwen3-8b", "q4_0", prompt)
    assert found is not None and found[1] == P and found[0].endswith(name)
    fresh = [device_storage_like(ko.HostCache(1024, H, d, 32, 3)) for _ in range(layers)]
    assert kv.load_session(found[0], "qwen3-8b", "q4_0", fresh) == tokens
    q = to_dev(ko.normal_f16(rng, (Hq, d)))
    ws = kv.decode_workspace(Hq, d)
    for a, b in zip(sts, fresh):
        oa, ob = torch.empty(Hq, d, device="cuda"), torch.empty(Hq, d, device="cuda")
        kv.launch_decode_attention_quant(a.view(), q, query_heads=Hq, scale=d ** -0.5, cache_length=P, output=oa, workspace=ws)
        kv.launch_decode_attention_quant(b.view(), q, query_heads=Hq, scale=d ** -0.5, cache_length=P, output=ob, workspace=ws)
        torch.cuda.synchronize()
        assert torch.equal(oa, ob)
    other_mode = [kv.AttentionLayerKvCacheStorage(1024, kv.KvCacheQuantMode.kQ8Fp16, kv_heads=H, head_dim=d, qblock=32) for _ in range(layers)]
    assert kv.load_session(found[0], "qwen3-8b", "q4_0", other_mode) is None
    assert kv.load_session(found[0], "another-model", "q4_0", fresh) is None
    too_small = [kv.AttentionLayerKvCacheStorage(512, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=d, qblock=32) for _ in range(layers)]
    with pytest.raises(kv.B200KvError):
        kv.load_session(found[0], "qwen3-8b", "q4_0", too_small)


@pytest.mark.parametrize("P,T,H,Hq,d", [(2048, 128, 4, 24, 256), (1500, 200, 8, 32, 128), (4096, 512, 1, 6, 256)])   # the last one: 6 splits
def test_suffix_attention_with_the_kv_range_split_over_ctas(cuda, P, T, H, Hq, d):
    """Few row tiles, long prefix: with room for partials in the workspace the tcgen05 launch splits every row
    tile's KV range over several CTAs and merges the partials; the result must match the unsplit launch and the oracle."""
    rng = np.random.default_rng(P + T)
    host = filled(rng, P + T, H, d, 32, 3, cap=P + T + 64, std=0.5)
    st = upload(host)
    q = (rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)
    gate = (rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)
    ref = host.suffix_ref(q, gate, P, d ** -0.5)
    plain = torch.full((T, Hq, d), float("nan"), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), to_dev(q), to_dev(gate), plain, kv.prefill_workspace(P + T, H, d), T, P,
                                     query_heads=Hq, scale=d ** -0.5)
    split = torch.full((T, Hq, d), float("nan"), device="cuda")
    ws = kv.prefill_workspace(P + T, H, d, token_count=T, query_heads=Hq)
    assert ws.numel() > kv.prefill_workspace(P + T, H, d).numel()
    kv.launch_suffix_attention_quant(st.view(), to_dev(q), to_dev(gate), split, ws, T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    assert np.max(np.abs(split.cpu().numpy() - ref)) <= TOL
    assert float((split - plain).abs().max()) <= 1e-4     # same tiles, merged in a different order


def test_suffix_chunks_back_to_back_with_launch_overlap(cuda):
    """With launch overlap on, the kernels of consecutive chunks (store, fp16 pre-pass, attention, merge) become resident
    while their predecessors still run and order themselves by their own dependency waits: the outputs of three chunks
    launched back to back must equal those of the serialised launches bit for bit."""
    rng = np.random.default_rng(77)
    P, T, H, Hq, d = 1024, 128, 4, 24, 256
    host = filled(rng, P, H, d, 32, 3, cap=P + 3 * T, std=0.5)
    w = to_dev((1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    chunks = [(to_dev(ko.normal_f16(rng, (T, H * d))), to_dev(ko.normal_f16(rng, (T, H * d))),
               to_dev((rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32)),
               to_dev((rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32))) for _ in range(3)]
    outs = {}
    for overlap in (0, 1):
        st = upload(host)
        ws = kv.prefill_workspace(P + 3 * T, H, d, token_count=T, query_heads=Hq)
        out = torch.full((3, T, Hq, d), float("nan"), device="cuda")
        kv.set_launch_overlap(overlap)
        try:
            for i, (k, v, q, gate) in enumerate(chunks):
                kv.launch_kv_store_quant(st.view(), k, v, w, T, P + i * T, rope_mode=kv.RopeMode.SECTIONED64)
                kv.launch_suffix_attention_quant(st.view(), q, gate, out[i], ws, T, P + i * T, query_heads=Hq, scale=d ** -0.5)
            torch.cuda.synchronize()
        finally:
            kv.set_launch_overlap(0)
        outs[overlap] = out.cpu()
    assert torch.isfinite(outs[1]).all()
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("P,T,H,Hq,d,prepared", [(2048, 128, 4, 24, 256, 2048), (1500, 200, 8, 32, 128, 1000), (640, 64, 4, 24, 256, 0)])
def test_suffix_attention_over_a_prefix_converted_ahead_on_a_second_stream(cuda, P, T, H, Hq, d, prepared):
    """b200kv_prefill_prepare converts the prefix to fp16 ahead of the chunk (here on a second stream, ordered by
    events, with launch overlap on); the attention call that is told so converts only the rest.  Two layers in turn
    on two workspaces, as a host pipelines them; every output must equal the plain call's bit for bit and match the oracle."""
    rng = np.random.default_rng(P + T + prepared)
    hosts = [filled(rng, P + T, H, d, 32, 3, cap=P + T + 64, std=0.5) for _ in range(2)]
    sts = [upload(h) for h in hosts]
    q = [(rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32) for _ in range(2)]
    gate = [(rng.standard_normal((T, Hq, d)) * 0.5).astype(np.float32) for _ in range(2)]
    plain = torch.full((2, T, Hq, d), float("nan"), device="cuda")
    ws = [kv.prefill_workspace(P + T, H, d, token_count=T, query_heads=Hq) for _ in range(2)]
    for l in range(2):
        kv.launch_suffix_attention_quant(sts[l].view(), to_dev(q[l]), to_dev(gate[l]), plain[l], ws[l], T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    for w in ws:
        w.fill_(0xFF)            # nothing of the plain calls' scratch may help (0xFFFF is a NaN in fp16)
    ahead = torch.full((2, T, Hq, d), float("nan"), device="cuda")
    qd, gd = [to_dev(x) for x in q], [to_dev(x) for x in gate]
    main, side = torch.cuda.Stream(), torch.cuda.Stream()
    done = [torch.cuda.Event() for _ in range(2)]
    kv.set_launch_overlap(1)
    try:
        with torch.cuda.stream(main):
            side.wait_stream(main)
            for l in range(2):
                kv.prepare_suffix_attention(sts[l].view(), prepared, P + T, ws[l], stream=side)
                done[l].record(side)
            for l in range(2):
                main.wait_event(done[l])
                kv.launch_suffix_attention_quant(sts[l].view(), qd[l], gd[l], ahead[l], ws[l], T, P, query_heads=Hq, scale=d ** -0.5,
                                                 prepared_rows=prepared)
        torch.cuda.synchronize()
    finally:
        kv.set_launch_overlap(0)
    assert torch.equal(ahead.cpu(), plain.cpu())
    for l in range(2):
        assert np.max(np.abs(ahead[l].cpu().numpy() - hosts[l].suffix_ref(q[l], gate[l], P, d ** -0.5))) <= TOL
    # more rows declared than the chunk can see, or a workspace that is too small, are refused
    with pytest.raises(kv.B200KvError):
        kv.prepare_suffix_attention(sts[0].view(), P + T + 1, P + T, ws[0])
    with pytest.raises(kv.B200KvError):
        kv.prepare_suffix_attention(sts[0].view(), 16, P + T, torch.empty(1024, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_quantized_suffix_errors_on_the_reference_recipe(cuda, kernel):
    """The reference's quantized-attention test recipe (tests/qwen3_quant_kv_attention_test.cpp:79-154; the same
    std::mt19937(42) stream, its host quantiser, fp16 against Q8-K+V caches) through the CUDA kernels: the error of
    the quantised cache against the fp16 one must come out where the reference measured it on its own GPU kernels and
    where the oracle puts it (tests/golden/quant_kv_attention_pin.json; first case: max-abs 0.001263, cosine
    0.999973 in the reference's record)."""
    import importlib.util
    import json
    from pathlib import Path

    golden = Path(__file__).parent / "golden"
    spec = importlib.util.spec_from_file_location("make_statistical_pin", golden / "make_statistical_pin.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    want = json.loads((golden / "quant_kv_attention_pin.json").read_text())["cases"]
    for case, (P, T, q, gate, k, v) in zip(want, gen.draw_cases(3)):
        outs = {}
        for mode in (0, 3):
            st = upload(gen.host_cache(P, T, k, v, mode))
            out = torch.full((T, 24, 256), float("nan"), device="cuda")
            ws = kv.prefill_workspace(P + T, 4, 256, token_count=T, query_heads=24) if kernel == "tcgen05" else None
            kv.launch_suffix_attention_quant(st.view(), to_dev(q), to_dev(gate), out, ws, T, P, query_heads=24, scale=1.0 / 16.0)
            torch.cuda.synchronize()
            outs[mode] = out.cpu().numpy()
        got = gen.metrics(outs[0], outs[3])
        ref = case["q8_kv"]
        print(f"{kernel} P={P} T={T}: max-abs {got['max_abs']:.6f} (oracle {ref['max_abs']:.6f}), MAE {got['mae']:.6f} ({ref['mae']:.6f}), "
              f"cos {got['cos']:.8f} ({ref['cos']:.8f})")
        assert abs(got["max_abs"] - ref["max_abs"]) <= 0.05 * ref["max_abs"] + 2e-5
        assert abs(got["mae"] - ref["mae"]) <= 0.05 * ref["mae"]
        assert abs(got["cos"] - ref["cos"]) <= 3e-6
