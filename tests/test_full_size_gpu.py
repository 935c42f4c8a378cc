"""GPU parity at the sizes the benchmark set names, through the C ABI, against the CPU oracle:
decode attention at 32,768 and 131,072 positions (plain and fused with the append), the 512-token suffix over an
8,192-token prefix on the tcgen05 kernel (with and without the KV split), the batched step over 64 seeded
lengths plus 16 sessions restored from a 4,096-token clone, and sequence-sharded decode with 8 ranks of which
7 are simulated (their partials are delivered beforehand; kernels that wait for each other are never launched
on one device), and decode attention at head_dim 256 with 24 query heads over 4 kv heads at both contexts.  Every case asserts max-abs <= 2e-3 and a relative L2 gate, and prints both errors."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_attention_close, assert_planes_equal, to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu
H, HQ, D = 8, 32, 128


def _long_cache(rng, length, capacity):
    host = ko.HostCache(capacity, H, D, 32, 3)
    chunk = 16384
    for base in range(0, length, chunk):
        n = min(chunk, length - base)
        host.append(ko.normal_f16(rng, (n, H * D)).astype(np.float32), ko.normal_f16(rng, (n, H * D)).astype(np.float32),
                    None, base, rope_mode=0)
    return host


@pytest.mark.parametrize("length", [32768, 131072])
@pytest.mark.parametrize("kernel", ["auto", "mma"])
def test_decode_attention_and_fused_step_at_benchmark_context(cuda, length, kernel):
    rng = np.random.default_rng(length)
    host = _long_cache(rng, length - 1, length + 64)       # length - 1 resident rows, the step appends the last one
    st = upload(host)
    assert kv.decode_kernel_kind(st.view(), HQ) == 1
    ws = kv.decode_workspace(HQ, D)
    kv.set_decode_kernel(1 if kernel == "mma" else 0)
    try:
        # plain attention over the resident rows
        q16 = ko.normal_f16(rng, (HQ, D))
        gate = rng.standard_normal((HQ, D)).astype(np.float32)
        ref, ref_g = host.decode_ref(q16.astype(np.float32), D ** -0.5, length - 1, gate)
        out = torch.full((HQ, D), float("nan"), device="cuda"); gated = torch.full((HQ, D), float("nan"), device="cuda")
        kv.launch_decode_attention_quant(st.view(), to_dev(q16), query_heads=HQ, scale=D ** -0.5, cache_length=length - 1,
                                         output=out, gate=to_dev(gate), gated_output=gated, workspace=ws)
        torch.cuda.synchronize()
        assert_attention_close(out.cpu().numpy(), ref, f"decode_attn[{kernel}] L={length - 1}")
        assert_attention_close(gated.cpu().numpy(), ref_g, f"decode_attn[{kernel}] gated L={length - 1}")
        # fused step: append the token at position length-1 (NeoX RoPE at its true position) and attend `length` rows
        kn, vn = ko.normal_f16(rng, (1, H * D)), ko.normal_f16(rng, (1, H * D))
        host.append(kn.astype(np.float32), vn.astype(np.float32), None, length - 1, rope_mode=1)
        ref2, _ = host.decode_ref(q16.astype(np.float32), D ** -0.5, length)
        state = kv.make_decode_state(length - 1)
        out2 = torch.full((HQ, D), float("nan"), device="cuda")
        kv.launch_decode_step(st.view(), to_dev(kn), to_dev(vn), to_dev(q16), query_heads=HQ, scale=D ** -0.5, decode_state=state,
                              rope_mode=kv.RopeMode.NEOX_FULL, output=out2, workspace=ws)
        torch.cuda.synchronize()
        assert_planes_equal(st, host, "row appended by the fused step")
        assert_attention_close(out2.cpu().numpy(), ref2, f"decode_step[{kernel}] L={length}")
    finally:
        kv.set_decode_kernel(0)


@pytest.mark.parametrize("split", [False, True])
def test_suffix_512_over_8192_on_the_tcgen05_kernel(cuda, split):
    P, T, Hk, Hq, d = 8192, 512, 4, 24, 256
    rng = np.random.default_rng(8192 + 512)
    host = ko.HostCache(P + T, Hk, d, 32, 3)
    host.append(ko.normal_f16(rng, (P + T, Hk * d)).astype(np.float32), ko.normal_f16(rng, (P + T, Hk * d)).astype(np.float32),
                None, 0, rope_mode=0)
    st = upload(host)
    q16 = ko.normal_f16(rng, (T, Hq, d))
    gate = rng.standard_normal((T, Hq, d)).astype(np.float32)
    ref = host.suffix_ref(q16.astype(np.float32), gate, P, d ** -0.5)
    ws = kv.prefill_workspace(P + T, Hk, d, token_count=T, query_heads=Hq) if split else kv.prefill_workspace(P + T, Hk, d)
    out = torch.full((T, Hq, d), float("nan"), device="cuda")
    kv.launch_suffix_attention_quant(st.view(), to_dev(q16), to_dev(gate), out, ws, T, P, query_heads=Hq, scale=d ** -0.5)
    torch.cuda.synchronize()
    # the tcgen05 kernel rounds the dequantised K/V and the weights to fp16 (11 bits): relative L2 gate 2e-3
    assert_attention_close(out.cpu().numpy(), ref, f"suffix tcgen05 {T} over {P} (kv split {split})", tol_rel=2.0e-3)


def test_batched_64_seeded_lengths_plus_16_restored_from_a_clone(cuda):
    rng = np.random.default_rng(42)
    lengths = [int(x) for x in rng.integers(512, 16385, size=64)] + [4096] * 16
    proto_host = _long_cache(rng, 4096, 4096 + 64)
    proto = upload(proto_host)
    hosts, sts = [], []
    for i, L in enumerate(lengths):
        if i < 64:
            h = _long_cache(rng, L, (L + 8 + 63) // 64 * 64)
            hosts.append(h); sts.append(upload(h))
        else:   # restored session: a device-to-device clone of the shared 4096-token prefix
            s = kv.AttentionLayerKvCacheStorage(4096 + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=D, qblock=32)
            s.clone_prefix_from(proto, 4096)
            hosts.append(proto_host); sts.append(s)
    S = len(lengths)
    q16 = ko.normal_f16(rng, (S, HQ, D))
    lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    ws = kv.decode_workspace(HQ, D, S)
    table = kv.view_table(S)
    for kernel in ("auto", "mma"):
        kv.set_decode_kernel(1 if kernel == "mma" else 0)
        try:
            out = torch.full((S, HQ, D), float("nan"), device="cuda")
            kv.launch_decode_attention_batched([s.view() for s in sts], table, lens, max(lengths), to_dev(q16), query_heads=HQ,
                                               scale=D ** -0.5, output=out, workspace=ws)
            torch.cuda.synchronize()
        finally:
            kv.set_decode_kernel(0)
        got = out.cpu().numpy()
        worst_abs = worst_rel = 0.0
        for i, h in enumerate(hosts):
            ref, _ = h.decode_ref(q16[i].astype(np.float32), D ** -0.5, lengths[i])
            diff = got[i] - ref
            worst_abs = max(worst_abs, float(np.max(np.abs(diff))))
            worst_rel = max(worst_rel, float(np.linalg.norm(diff) / np.linalg.norm(ref)))
        print(f"[parity] batched[{kernel}] 64 + 16 sessions: worst max_abs {worst_abs:.3e} worst rel_l2 {worst_rel:.3e}")
        assert worst_abs <= 2.0e-3 and worst_rel <= 1.0e-3


def test_sequence_sharded_decode_with_8_ranks_7_of_them_simulated(cuda):
    from miinfer_b200.partition import shard_range

    L, world = 131072, 8
    rng = np.random.default_rng(131072 + 8)
    host = _long_cache(rng, L, L)
    st = upload(host)
    q16 = ko.normal_f16(rng, (HQ, D))
    q = to_dev(q16)
    want, _ = host.decode_ref(q16.astype(np.float32), D ** -0.5, L)
    ws = kv.decode_workspace(HQ, D)
    words_per_rank = HQ * (D + 2)
    sequence = 5      # any call number: both the slot (sequence & 1) and the tag of the words derive from it
    own = torch.zeros(2 * world * words_per_rank, dtype=torch.int64, device="cuda")
    peers = [own] + [torch.zeros_like(own) for _ in range(world - 1)]
    for r in range(1, world):    # what ranks 1..7 would have stored into rank 0's buffer
        b, e = shard_range(L, r, world)
        mine = kv.packed_partial(HQ, D, 1)
        pm, pl, pa = kv.partial_views(mine[0], HQ, D)
        kv.launch_decode_partials(st.view(), q, query_heads=HQ, scale=D ** -0.5, range_begin=b, range_end=e,
                                  part_m=pm, part_l=pl, part_acc=pa, workspace=ws)
        torch.cuda.synchronize()
        slot = own[((sequence & 1) * world + r) * words_per_rank:((sequence & 1) * world + r + 1) * words_per_rank].view(HQ, D + 2)
        slot[:, :D] = kv.exchange_words(pa.view(HQ, D), sequence)
        slot[:, D] = kv.exchange_words(pm, sequence)
        slot[:, D + 1] = kv.exchange_words(pl, sequence)
    ex = kv.Exchange.from_pointers([t.data_ptr() for t in peers], 0)
    b0, e0 = shard_range(L, 0, world)
    out = torch.full((HQ, D), float("nan"), device="cuda")
    kv.launch_decode_attention_sharded(st.view(), q, ex, query_heads=HQ, scale=D ** -0.5, range_begin=b0, range_end=e0,
                                       phase=sequence, output=out, workspace=ws)
    torch.cuda.synchronize()
    assert_attention_close(out.cpu().numpy(), want, "sharded decode, 8 ranks (7 simulated), L=131072")
    assert int(own.abs().sum()) == 0      # consumed words are zero again


@pytest.mark.parametrize("length", [32768, 131072])
def test_decode_attention_head_dim_256_at_benchmark_context(cuda, length):
    """The reference's own geometry (24 query heads over 4 kv heads, head_dim 256, q8_0 blocks) on the tcgen05 stage-1
    kernel for head_dim 256, at the contexts the benchmark set names; also through the fused-step entry point, which for
    this geometry is the store kernel followed by the attention."""
    Hk, Hq, d = 4, 24, 256
    rng = np.random.default_rng(length + d)
    host = ko.HostCache(length + 64, Hk, d, 32, 3)
    chunk = 16384
    for base in range(0, length - 1, chunk):
        n = min(chunk, length - 1 - base)
        host.append(ko.normal_f16(rng, (n, Hk * d)).astype(np.float32), ko.normal_f16(rng, (n, Hk * d)).astype(np.float32), None, base, rope_mode=0)
    st = upload(host)
    assert kv.decode_kernel_kind(st.view(), Hq) == 2
    ws = kv.decode_workspace(Hq, d)
    q16 = ko.normal_f16(rng, (Hq, d))
    gate = rng.standard_normal((Hq, d)).astype(np.float32)
    ref, ref_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, length - 1, gate)
    out = torch.full((Hq, d), float("nan"), device="cuda"); gated = torch.full((Hq, d), float("nan"), device="cuda")
    kv.launch_decode_attention_quant(st.view(), to_dev(q16), query_heads=Hq, scale=d ** -0.5, cache_length=length - 1,
                                     output=out, gate=to_dev(gate), gated_output=gated, workspace=ws)
    torch.cuda.synchronize()
    assert_attention_close(out.cpu().numpy(), ref, f"decode_attn[d=256 tcgen05] L={length - 1}")
    assert_attention_close(gated.cpu().numpy(), ref_g, f"decode_attn[d=256 tcgen05] gated L={length - 1}")
    kn, vn = ko.normal_f16(rng, (1, Hk * d)), ko.normal_f16(rng, (1, Hk * d))
    w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    host.append(kn.astype(np.float32), vn.astype(np.float32), w, length - 1, rope_mode=2)
    ref2, _ = host.decode_ref(q16.astype(np.float32), d ** -0.5, length)
    state = kv.make_decode_state(length - 1)
    out2 = torch.full((Hq, d), float("nan"), device="cuda")
    kv.launch_decode_step(st.view(), to_dev(kn), to_dev(vn), to_dev(q16), query_heads=Hq, scale=d ** -0.5, decode_state=state,
                          k_norm_weight=to_dev(w), rope_mode=kv.RopeMode.SECTIONED64, output=out2, workspace=ws)
    torch.cuda.synchronize()
    assert_planes_equal(st, host, "row appended by the step (head_dim 256)")
    assert_attention_close(out2.cpu().numpy(), ref2, f"decode_step[d=256] L={length}")
