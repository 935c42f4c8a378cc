"""CPU tests: pin the oracle (oracle/kv_oracle.c) to the reference.

1. against outputs of the reference's own host primitives compiled in place
   (tests/golden/ref_host_primitives.npz, made by tests/golden/make_golden.py);
2. against the reference's stored traces for the KV path
   (tests/golden/m4a4_four_position.npz, m4b_layers.npz) -- the same vectors its
   tests/qwen3_kv_cache_test.cpp checks, at far tighter tolerances;
3. internal consistency: quantizer contract, split-K replica vs two-pass
   reference, merge associativity, snapshot layout, token hash.
"""
from pathlib import Path

import numpy as np
import pytest

import kvoracle as ko

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def ref_prims():
    return np.load(GOLD / "ref_host_primitives.npz")


@pytest.fixture(scope="module")
def four_pos():
    return np.load(GOLD / "m4a4_four_position.npz")


def test_half_to_float_matches_reference_all_patterns(ref_prims):
    bits = np.arange(65536, dtype=np.uint16)
    ours = ko.half_to_float(bits)
    ref = ref_prims["fp16_all"]
    nan = np.isnan(ref)   # NaN payloads are quieted by the float return through ctypes, so compare NaN-ness
    assert np.array_equal(np.isnan(ours), nan) and nan.sum() == 2046
    assert np.array_equal(ours.view(np.uint32)[~nan], ref.view(np.uint32)[~nan])
    # and numpy's IEEE half agrees
    assert np.array_equal(ours.view(np.uint32)[~nan], bits.view(np.float16).astype(np.float32).view(np.uint32)[~nan])


def test_float_to_half_rn_matches_ieee():
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 10,
        (rng.standard_normal(50000) * 1e-6).astype(np.float32),   # subnormal halves
        (rng.standard_normal(20000) * 7e4).astype(np.float32),    # overflow to inf
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 5.9604645e-8, 2.9802322e-8, 2.98023223876953125e-8,
                  np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.00146484375], np.float32),
    ])
    ours = ko.float_to_half(x)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(ours, ref)
    # round trip of every finite half is the identity
    bits = np.arange(65536, dtype=np.uint16)
    f = ko.half_to_float(bits)
    finite = np.isfinite(f)
    assert np.array_equal(ko.float_to_half(f[finite]), bits[finite])


def test_pinned_sincos_is_correctly_rounded_enough():
    rng = np.random.default_rng(3)
    angles = np.concatenate([rng.uniform(0, 131072, 20000), rng.uniform(0, 8, 5000), [0.0, 1.0, 131071.0]]).astype(np.float32)
    worst = 0.0
    for a in angles:
        s, c = ko.sincos_pinned(float(a))
        worst = max(worst, abs(s - np.sin(np.float64(a))), abs(c - np.cos(np.float64(a))))
    assert worst <= 6.0e-8  # within one fp32 rounding of the exact value


@pytest.mark.parametrize("d", [128, 256])
def test_neox_rope_matches_reference_primitive(ref_prims, d):
    x = ref_prims[f"rope_in_{d}"]
    for pos in (0, 1, 7, 1000, 32767, 131071):
        ref = ref_prims[f"rope_out_{d}_{pos}"]
        libm = ko.rope_heads(x, pos, 1.0e6, rope_mode=1, trig_mode=0)
        assert np.array_equal(libm, ref), f"libm-trig RoPE differs from rope_qwen3_reference at pos {pos}"
        pinned = ko.rope_heads(x, pos, 1.0e6, rope_mode=1, trig_mode=1)
        assert np.max(np.abs(pinned - ref)) <= 1.0e-6


def test_neox_rope_matches_stored_traces(four_pos):
    for p in range(4):
        for trig in (0, 1):
            k = ko.rope_heads(four_pos[f"k_normed_{p}"], p, 1.0e6, 1, trig)
            q = ko.rope_heads(four_pos[f"q_normed_{p}"], p, 1.0e6, 1, trig)
            assert np.max(np.abs(k - four_pos[f"k_rope_{p}"])) <= 4e-6   # reference gate: 2.5e-2
            assert np.max(np.abs(q - four_pos[f"q_rope_{p}"])) <= 4e-6
        assert np.array_equal(four_pos[f"cache_k_{p}"], four_pos[f"k_rope_{p}"])


def test_sectioned_rope_is_neox_on_first_64_dims():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 256), dtype=np.float32)
    pos = 777
    y = ko.rope_heads(x, pos, 1.0e7, rope_mode=2, trig_mode=0)
    assert np.array_equal(y[:, 64:], x[:, 64:])
    step = np.float32(np.power(np.float32(1.0e7), np.float32(-2.0 / 64.0)))
    for i in (0, 1, 5, 31):
        a = np.float32(pos)
        for _ in range(i):
            a = np.float32(a * step)
        c, s = np.cos(a, dtype=np.float32), np.sin(a, dtype=np.float32)
        np.testing.assert_allclose(y[:, i], x[:, i] * c - x[:, i + 32] * s, atol=2e-6)
        np.testing.assert_allclose(y[:, i + 32], x[:, i] * s + x[:, i + 32] * c, atol=2e-6)


def test_softmax_and_fp32_attention_match_stored_traces(four_pos, ref_prims):
    # softmax_reference (double denominator) == oracle's two-pass decode with identity K/V handling:
    for n in (1, 5, 4097):
        s_in, s_out = ref_prims[f"softmax_in_{n}"], ref_prims[f"softmax_out_{n}"]
        m = s_in.max()
        den = np.sum(np.exp((s_in - m).astype(np.float64)))
        ours = (np.exp((s_in - m).astype(np.float64)) / den).astype(np.float32)
        assert np.array_equal(ours, s_out)
    # model-free attention KAT: fp16 cache of the traced K/V rows, q_rope as the query
    cache = ko.HostCache(capacity=8, kv_heads=8, head_dim=128, qblock=128, quant_mode=0)
    for p in range(4):
        cache.key_f16[:, p, :] = ko.float_to_half(four_pos[f"cache_k_{p}"])
        cache.value_f16[:, p, :] = ko.float_to_half(four_pos[f"cache_v_{p}"])
        out, _ = cache.decode_ref(four_pos[f"q_rope_{p}"], 1.0 / np.sqrt(128.0), p + 1)
        ref = four_pos[f"attention_output_{p}"]
        # the trace holds fp32 K/V and an fp16-materialised output; ours stores K/V as fp16
        assert np.max(np.abs(out - ref)) <= 1.5e-3, p   # reference gate: 2.0e-2
        out2, _ = cache.decode_splitk(four_pos[f"q_rope_{p}"], 1.0 / np.sqrt(128.0), p + 1, 4)
        assert np.max(np.abs(out2 - out)) <= 1e-6


def test_deeper_layer_traces_position_zero():
    g = np.load(GOLD / "m4b_layers.npz")
    for layer in (6, 35):
        k = ko.rope_heads(g[f"k_normed_{layer}"], 0, 1.0e6, 1, 1)
        assert np.array_equal(k, g[f"k_normed_{layer}"])  # position 0 is the identity rotation
        np.testing.assert_allclose(g[f"k_rope_{layer}"], g[f"k_normed_{layer}"], atol=1e-6)
        cache = ko.HostCache(4, 8, 128, 128, 0)
        cache.key_f16[:, 0, :] = ko.float_to_half(g[f"k_rope_{layer}"])
        cache.value_f16[:, 0, :] = ko.float_to_half(g[f"v_reshape_{layer}"])
        out, _ = cache.decode_ref(g[f"q_rope_{layer}"], 1.0 / np.sqrt(128.0), 1)
        scale = np.maximum(1.0, np.abs(g[f"attention_output_{layer}"]))
        assert np.max(np.abs(out - g[f"attention_output_{layer}"]) / scale) <= 2e-3


def test_rms_norm_tree_close_to_reference_double_sum(ref_prims):
    # the store kernel sums squares in an fp32 tree, the host primitive in double: same value to fp32 noise
    x, w, ref = ref_prims["rms_in"], ref_prims["rms_w"], ref_prims["rms_out"]
    cache = ko.HostCache(4, 1, 256, 256, 0)
    cache.append(x[None, :], x[None, :], w, 0, rope_mode=0)
    got = ko.half_to_float(cache.key_f16[0, 0])
    np.testing.assert_allclose(got, ref, rtol=1.5e-3, atol=1e-6)  # fp16 storage dominates


# ---- quantizer contract ---------------------------------------------------------

def test_quantizer_half_even_clamp_and_zero_block():
    q, s = ko.quantize_block(np.zeros(32, np.float32))
    assert not q.any() and s == ko.float_to_half(np.array([1.0], np.float32))[0]   # zero block -> scale 1.0
    # ties: amax = 127 makes scale exactly 1, so x.5 values expose the rounding mode
    x = np.zeros(32, np.float32)
    x[0], x[1], x[2], x[3], x[4], x[5] = 127.0, 0.5, 1.5, 2.5, -0.5, -2.5
    q, s = ko.quantize_block(x, 0)
    assert list(q[:6]) == [127, 0, 2, 2, 0, -2]            # round-half-to-even (store kernel)
    q1, _ = ko.quantize_block(x, 1)
    assert list(q1[:6]) == [127, 1, 2, 3, -1, -3]          # half-away (the reference's host quantizers)
    # dequantised error bound: |x - q*scale_f32| <= scale/2
    rng = np.random.default_rng(1)
    for _ in range(200):
        x = rng.standard_normal(32).astype(np.float32) * rng.uniform(1e-3, 50)
        q, s = ko.quantize_block(x, 0)
        scale = np.abs(x).max() / np.float32(127.0)
        assert np.all(np.abs(x - q.astype(np.float32) * scale) <= scale * 0.5 * (1 + 1e-5))
        assert q.min() >= -128 and q.max() <= 127 and np.abs(q).max() == 127
        assert s == ko.float_to_half(np.array([scale], np.float32))[0]


@pytest.mark.parametrize("d,qb,mode", [(128, 32, 3), (256, 256, 3), (256, 32, 1), (128, 128, 2), (128, 32, 0)])
def test_append_layout_and_untouched_slots(d, qb, mode):
    rng = np.random.default_rng(11)
    H, cap, T, base = 2, 16, 3, 5
    cache = ko.HostCache(cap, H, d, qb, mode)
    k = ko.normal_f16(rng, (T, H * d)).astype(np.float32)
    v = ko.normal_f16(rng, (T, H * d)).astype(np.float32)
    cache.append(k, v, None, base, rope_mode=1 if d == 128 else 2)
    for name, plane in cache.planes().items():
        touched = np.zeros(cap, bool)
        touched[base:base + T] = True
        assert not plane[:, ~touched].any(), f"{name}: slots outside [base, base+T) were written"
        assert plane[:, touched].any()
    with pytest.raises(ValueError):
        cache.append(k, v, None, cap - 1, rope_mode=0)   # invalid append must be refused
    # V rows are quantised without rotation: check one block by hand
    if mode in (2, 3):
        q, s = ko.quantize_block(v[1].reshape(H, d)[1, :qb], 0)
        assert np.array_equal(cache.value_q8[1, base + 1, :qb], q) and cache.value_scales[1, base + 1, 0] == s


# ---- attention consistency ---------------------------------------------------------

def _filled_cache(rng, L, H, d, qb, mode, cap=None):
    cache = ko.HostCache(cap or L + 3, H, d, qb, mode)
    k = ko.normal_f16(rng, (L, H * d)).astype(np.float32)
    v = ko.normal_f16(rng, (L, H * d)).astype(np.float32)
    cache.append(k, v, None, 0, rope_mode=0)
    return cache


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_splitk_replica_matches_two_pass_reference(mode):
    rng = np.random.default_rng(21 + mode)
    cache = _filled_cache(rng, 333, 2, 128, 32, mode)
    q = ko.normal_f16(rng, (8, 128)).astype(np.float32)
    gate = rng.standard_normal((8, 128)).astype(np.float32)
    ref, ref_g = cache.decode_ref(q, 128 ** -0.5, 333, gate)
    for splits in (1, 4, 7, 64):
        out, out_g = cache.decode_splitk(q, 128 ** -0.5, 333, splits, gate)
        assert np.max(np.abs(out - ref)) <= 2e-6 and np.max(np.abs(out_g - ref_g)) <= 2e-6
    # probabilities sum to one: attention over constant V returns that constant
    if mode == 0:
        cache.value_f16[:] = ko.float_to_half(np.array([0.75], np.float32))[0]
        out, _ = cache.decode_ref(q, 128 ** -0.5, 333)
        np.testing.assert_allclose(out, 0.75, atol=1e-6)


def test_merge_is_associative_over_shards():
    rng = np.random.default_rng(31)
    cache = _filled_cache(rng, 1000, 2, 128, 32, 3)
    q = ko.normal_f16(rng, (8, 128)).astype(np.float32)
    ref, _ = cache.decode_ref(q, 128 ** -0.5, 1000)
    # 4 sequence shards, each reduced to one partial, then merged == full attention
    parts = []
    for r in range(4):
        m, l, acc = cache.decode_partials(q, 128 ** -0.5, r * 250, (r + 1) * 250, 3)
        # reduce the 3 local splits to one partial by the same rule
        gm = m.max(axis=0)
        a = np.exp(m - gm)
        parts.append((gm, (l * a).sum(0), (acc * a[:, :, None]).sum(0)))
    m = np.stack([p[0] for p in parts]); l = np.stack([p[1] for p in parts]); acc = np.stack([p[2] for p in parts])
    out, _ = ko.merge_partials(m, l, acc)
    assert np.max(np.abs(out - ref)) <= 2e-6
    # an empty shard (m=-inf, l=0) does not disturb the merge
    m2 = np.concatenate([m, np.full((1, 8), -np.inf, np.float32)])
    l2 = np.concatenate([l, np.zeros((1, 8), np.float32)])
    acc2 = np.concatenate([acc, np.zeros((1, 8, 128), np.float32)])
    out2, _ = ko.merge_partials(m2, l2, acc2)
    assert np.array_equal(out2, out)


def test_suffix_is_causal_and_matches_decode():
    rng = np.random.default_rng(41)
    P, T, H, Hq, d = 40, 6, 2, 4, 256
    cache = _filled_cache(rng, P + T, H, d, 32, 3, cap=P + T)
    q = ko.normal_f16(rng, (T, Hq, d)).astype(np.float32)
    gate = rng.standard_normal((T, Hq, d)).astype(np.float32)
    out = cache.suffix_ref(q, gate, P, d ** -0.5)
    for t in range(T):
        _, ref_g = cache.decode_ref(q[t], d ** -0.5, P + t + 1, gate[t])
        assert np.array_equal(out[t], ref_g)
    out_k = cache.suffix_splitk(q, gate, P, d ** -0.5, 32)
    assert np.max(np.abs(out_k - out)) <= 2e-6
    # mutation: a wrong base position must be visible (the reference's own mutation test idea)
    assert np.max(np.abs(cache.suffix_ref(q, gate, P - 1, d ** -0.5) - out)) > 1e-3


# ---- snapshot layout & prefix identity ---------------------------------------------

@pytest.mark.parametrize("mode,qb", [(0, 256), (1, 256), (2, 32), (3, 32), (3, 256)])
def test_snapshot_layout_and_round_trip(mode, qb):
    rng = np.random.default_rng(51)
    H, d, cap, tokens = 4, 256, 37, 19
    cache = _filled_cache(rng, cap, H, d, qb, mode, cap=cap)
    nblk = d // qb
    k_rec = tokens * (d + 2 * nblk) if mode in (1, 3) else tokens * d * 2
    v_rec = tokens * (d + 2 * nblk) if mode in (2, 3) else tokens * d * 2
    assert cache.raw_tokens_bytes(tokens) == H * (k_rec + v_rec)
    if mode == 3 and qb == 256:   # the reference's own formula, kv_cache.cpp:222: 2*tokens*kv_heads*(head_dim+2)
        assert cache.raw_tokens_bytes(tokens) == 2 * tokens * H * (d + 2)
    blob = cache.download_raw(tokens)
    if mode in (1, 3):   # head 1's int8 slice starts one record after head 0's
        assert np.array_equal(blob[k_rec:k_rec + tokens * d].view(np.int8).reshape(tokens, d), cache.key_q8[1, :tokens])
        sc = blob[k_rec + tokens * d:2 * k_rec].view(np.uint16).reshape(tokens, nblk)
        assert np.array_equal(sc, cache.key_scales[1, :tokens])
    other = ko.HostCache(cap + 9, H, d, qb, mode)
    other.upload_raw(blob, tokens)
    for name, plane in cache.planes().items():
        assert np.array_equal(other.planes()[name][:, :tokens], plane[:, :tokens])
        assert not other.planes()[name][:, tokens:].any()


def test_token_hash_is_per_token_fnv():
    h = 0xcbf29ce484222325
    for t in (14990, 42, 31415, 2718):
        h = ((h ^ t) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    assert ko.token_sequence_hash([14990, 42, 31415, 2718]) == h
    assert ko.token_sequence_hash([]) == 0xcbf29ce484222325
    assert ko.token_sequence_hash([1, 2]) != ko.token_sequence_hash([2, 1])
