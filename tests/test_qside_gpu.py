"""GPU parity of the operators either side of the KV path in a step: the query-side split / RMSNorm / RoPE
(bit-exact against the oracle, and bit-identical to what the append kernel does to a key at the same position),
the Q8_1 re-quantisation of the decode output, and the device-side decode-state advance."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,heads,rope,norm,tokens,base", [
    (256, 24, 2, True, 70, 8192),       # the hybrid model's shape: sectioned RoPE on the first 64 dims, q-norm
    (128, 32, 1, False, 5, 131000),     # NeoX full width, no norm, far positions
    (128, 32, 1, True, 1, 4096),
    (256, 6, 0, True, 3, 0),
])
def test_q_split_norm_rope_is_bit_exact(cuda, d, heads, rope, norm, tokens, base):
    rng = np.random.default_rng(d + heads + tokens)
    qfull = rng.standard_normal((tokens, heads, 2 * d)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32) if norm else None
    want_q, want_g = ko.q_split_norm_rope(qfull, w, base, rope_mode=rope)
    q = torch.full((tokens, heads, d), float("nan"), device="cuda")
    g = torch.full((tokens, heads, d), float("nan"), device="cuda")
    kv.launch_q_split_norm_rope(to_dev(qfull), None if w is None else to_dev(w), q, g, tokens, base, heads=heads, head_dim=d,
                                rope_mode=kv.RopeMode(rope))
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy().view(np.uint32), want_q.view(np.uint32))
    assert np.array_equal(g.cpu().numpy().view(np.uint32), want_g.view(np.uint32))
    # fp16 input and output: the same arithmetic on the upcast values, rounded to nearest on the way out
    q16in = qfull.astype(np.float16)
    want_q2, _ = ko.q_split_norm_rope(q16in.astype(np.float32), w, base, rope_mode=rope)
    qh = torch.zeros((tokens, heads, d), device="cuda", dtype=torch.float16)
    kv.launch_q_split_norm_rope(to_dev(q16in), None if w is None else to_dev(w), qh, None, tokens, base, heads=heads, head_dim=d,
                                rope_mode=kv.RopeMode(rope))
    torch.cuda.synchronize()
    assert np.array_equal(qh.cpu().numpy().view(np.uint16), ko.float_to_half(want_q2))


def test_query_and_key_at_one_position_are_rotated_by_the_same_bits(cuda):
    """The same row through the query-side kernel and through the append kernel (fp16 cache, so that the rotated
    key is stored unquantised) must give the same fp16 bits, from host arguments and from device-side state."""
    rng = np.random.default_rng(4)
    d, H, pos = 256, 4, 7777
    row = rng.standard_normal((1, H, d)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    st = kv.AttentionLayerKvCacheStorage(8192, kv.KvCacheQuantMode.kFp16Fp16, kv_heads=H, head_dim=d)
    state = kv.make_decode_state(pos)
    kv.launch_kv_store_quant(st.view(), to_dev(row.reshape(1, H * d)), to_dev(row.reshape(1, H * d)), to_dev(w), 1, 0,
                             rope_mode=kv.RopeMode.SECTIONED64, decode_state=state)
    qfull = np.concatenate([row, np.zeros_like(row)], axis=2)
    q = torch.zeros((1, H, d), device="cuda", dtype=torch.float16)
    kv.launch_q_split_norm_rope(to_dev(qfull), to_dev(w), q, None, 1, 0, heads=H, head_dim=d, rope_mode=kv.RopeMode.SECTIONED64,
                                decode_state=state)
    torch.cuda.synchronize()
    assert torch.equal(q[0].view(torch.int16), st.key_cache[:, pos, :].view(torch.int16))


@pytest.mark.parametrize("d,H,Hq,L,splits,path", [
    (128, 8, 32, 3000, 0, "auto"), (128, 8, 32, 3000, 0, "mma"), (128, 8, 32, 200, 1, "auto"), (128, 8, 32, 200, 1, "mma"),
    (256, 4, 24, 700, 0, "generic"), (128, 8, 32, 700, 0, "generic")])
def test_decode_output_requantised_to_q8_1_blocks(cuda, d, H, Hq, L, splits, path):
    """gated_output_q8 is the Q8_1 form of the gated output the same launch writes: bit-equal to the oracle's
    block quantiser (half away from zero, +-127, d and s in fp16) applied to that fp32 output."""
    rng = np.random.default_rng(L + d)
    host = ko.HostCache((L + 7) // 8 * 8, H, d, 32, 3)
    host.append(ko.normal_f16(rng, (L, H * d)).astype(np.float32), ko.normal_f16(rng, (L, H * d)).astype(np.float32), None, 0, rope_mode=0)
    st = upload(host)
    q16 = ko.normal_f16(rng, (Hq, d))
    gate = rng.standard_normal((Hq, d)).astype(np.float32)
    ws = kv.decode_workspace(Hq, d)
    kv.set_decode_kernel(1 if path == "mma" else 0)
    try:
        for g in (to_dev(gate), None):
            gated = torch.full((Hq, d), float("nan"), device="cuda")
            blocks = kv.q8_1_blocks(Hq, d)
            kv.launch_decode_attention_quant(st.view(), to_dev(q16), query_heads=Hq, scale=d ** -0.5, cache_length=L, gate=g,
                                             gated_output=gated, gated_output_q8=blocks, workspace=ws,
                                             num_splits=splits | (kv.FORCE_GENERIC if path == "generic" else 0))
            torch.cuda.synchronize()
            want = ko.quantize_q8_1(gated.cpu().numpy())
            assert np.array_equal(blocks.cpu().numpy(), want)
            # the Q8_1 output alone is a valid request too (the reference launcher accepts any one of the three outputs)
            only = kv.q8_1_blocks(Hq, d)
            kv.launch_decode_attention_quant(st.view(), to_dev(q16), query_heads=Hq, scale=d ** -0.5, cache_length=L, gate=g,
                                             gated_output_q8=only, workspace=ws,
                                             num_splits=splits | (kv.FORCE_GENERIC if path == "generic" else 0))
            torch.cuda.synchronize()
            assert torch.equal(only, blocks)
    finally:
        kv.set_decode_kernel(0)
    ref, ref_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, L, None)
    assert np.max(np.abs(gated.cpu().numpy() - ref)) <= 2e-3


def test_decode_state_advance_matches_the_reference_bookkeeping(cuda):
    out_dev = torch.zeros(6, dtype=torch.int32, device="cuda")
    out_host = np.zeros(6, np.uint32)
    state_dev = kv.make_decode_state(100)
    state_dev[4] = 5          # max_generated
    state_host = np.zeros(16, np.uint32); state_host[1] = 100; state_host[4] = 5
    for token in (11, 22, 151645, 44, 55, 66, 77, 88):     # an end-of-text token, then past max_generated and past the capacity
        state_dev[0] = token; state_host[0] = token
        kv.launch_decode_state_advance(state_dev, out_dev)
        ko.decode_state_advance(state_host, out_host)
        torch.cuda.synchronize()
        assert np.array_equal(state_dev.cpu().numpy().view(np.uint32), state_host)
        assert np.array_equal(out_dev.cpu().numpy().view(np.uint32), out_host)
    assert state_host[1] == 108 and state_host[2] == 8 and state_host[3] == 1
