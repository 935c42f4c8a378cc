"""GPU parity: the fused append kernel against the oracle, BIT-EXACT (int8
quants, fp16 scales, fp16 passthrough rows), through the C ABI."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_planes_equal, device_storage_like, to_dev
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu

# (head_dim, kv_heads, qblock, mode, rope_mode, k_norm, dtype)
CASES = [
    (128, 8, 32, 3, 1, False, np.float16),    # the Qwen3-8B-shaped workloads: q8_0 blocks, NeoX RoPE, fp16 in
    (256, 4, 32, 3, 2, True, np.float16),     # config 3: sectioned RoPE + K RMSNorm
    (256, 4, 256, 3, 2, True, np.float32),    # the reference's own format: one scale per row, fp32 in
    (256, 4, 256, 1, 2, True, np.float32),    # Q8 K + fp16 V
    (256, 4, 256, 2, 2, True, np.float32),    # fp16 K + Q8 V
    (128, 8, 128, 0, 1, False, np.float16),   # fp16/fp16
    (128, 2, 32, 3, 0, False, np.float32),    # no RoPE
    (128, 8, 32, 3, 1, True, np.float32),
    (128, 12, 32, 3, 1, True, np.float16),    # more heads than one pass of the kernel takes (8 + 4)
    (256, 6, 32, 3, 2, True, np.float16),     # the same at head_dim 256 (4 + 2)
    (128, 3, 128, 1, 1, False, np.float32),   # a ragged pass with one scale per row and an fp16 side
]


def run_case(d, H, qb, mode, rope, norm, dtype, T, base, cap, seed, theta=1.0e6, via_state=None):
    rng = np.random.default_rng(seed)
    k = ko.normal_f16(rng, (T, H * d)) if dtype == np.float16 else rng.standard_normal((T, H * d), dtype=np.float32) * 1.7
    v = ko.normal_f16(rng, (T, H * d)) if dtype == np.float16 else rng.standard_normal((T, H * d), dtype=np.float32) * 0.3
    w = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32) if norm else None
    host = ko.HostCache(cap, H, d, qb, mode)
    host.append(k.astype(np.float32), v.astype(np.float32), w, base, rope_mode=rope, theta=theta, trig_mode=1)
    st = device_storage_like(host)
    kd, vd = to_dev(k), to_dev(v)
    wd = None if w is None else to_dev(w)
    view = st.view()
    if via_state == "prefill":
        state = kv.make_prefill_state(base, T)
        kv.launch_kv_store_quant(view, kd, vd, wd, T, 0, rope_mode=kv.RopeMode(rope), theta=theta, prefill_state=state)
    elif via_state == "decode":
        state = kv.make_decode_state(base)
        kv.launch_kv_store_quant(view, kd, vd, wd, 1, 0, rope_mode=kv.RopeMode(rope), theta=theta, decode_state=state)
    else:
        kv.launch_kv_store_quant(view, kd, vd, wd, T, base, rope_mode=kv.RopeMode(rope), theta=theta)
    torch.cuda.synchronize()
    assert_planes_equal(st, host, f"d={d} qb={qb} mode={mode} rope={rope} norm={norm} T={T} base={base}")
    return st, host


@pytest.mark.parametrize("d,H,qb,mode,rope,norm,dtype", CASES)
def test_append_bit_exact(cuda, d, H, qb, mode, rope, norm, dtype):
    run_case(d, H, qb, mode, rope, norm, dtype, T=37, base=5, cap=64, seed=100 + d + mode)
    run_case(d, H, qb, mode, rope, norm, dtype, T=1, base=63, cap=64, seed=7)      # last slot


def test_append_long_positions_bit_exact(cuda):
    # large positions stress the trig reduction: positions near 32K and 128K
    run_case(128, 8, 32, 3, 1, False, np.float16, T=64, base=32768 - 64, cap=32768, seed=1)
    run_case(128, 8, 32, 3, 1, False, np.float16, T=16, base=131072 - 16, cap=131072, seed=2)
    run_case(256, 4, 32, 3, 2, True, np.float16, T=512, base=8192, cap=8704, seed=3, theta=1.0e7)   # config-3 chunk


def test_append_positions_from_device_state(cuda):
    run_case(256, 4, 256, 3, 2, True, np.float32, T=9, base=21, cap=40, seed=4, via_state="prefill")
    run_case(128, 8, 32, 3, 1, False, np.float16, T=1, base=17, cap=40, seed=5, via_state="decode")


def test_append_edge_values(cuda):
    # zero rows (scale 1.0), ties at .5 (half-even), a lone huge value, denormal-ish rows
    d, H = 128, 2
    k = np.zeros((4, H * d), np.float32)
    v = np.zeros((4, H * d), np.float32)
    v[1, :32] = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -2.5, 63.5, -63.5] + [0.0] * 24, np.float32)
    v[2, 5] = 60000.0
    v[3, :] = 1.0e-7
    k[1:] = v[1:]
    host = ko.HostCache(8, H, d, 32, 3)
    host.append(k, v, None, 2, rope_mode=0)
    st = device_storage_like(host)
    kv.launch_kv_store_quant(st.view(), to_dev(k), to_dev(v), None, 4, 2, rope_mode=kv.RopeMode.NONE)
    torch.cuda.synchronize()
    assert_planes_equal(st, host, "edge values")
    assert list(st.value_cache_q8[0, 3, :8].cpu().numpy()) == [127, 0, 2, 2, 0, -2, 64, -64]


def test_append_rejects_out_of_range_and_keeps_other_slots(cuda):
    st = kv.AttentionLayerKvCacheStorage(16, kv.KvCacheQuantMode.kQ8Q8, kv_heads=2, head_dim=128, qblock=32)
    x = torch.randn(4, 256, device="cuda", dtype=torch.float16)
    with pytest.raises(kv.B200KvError) as e:
        kv.launch_kv_store_quant(st.view(), x, x, None, 4, 14, rope_mode=kv.RopeMode.NEOX_FULL)
    assert e.value.status == -6
    # with a device-side position the kernel itself drops rows that would leave the cache
    state = kv.make_prefill_state(14, 4)
    kv.launch_kv_store_quant(st.view(), x, x, None, 4, 0, rope_mode=kv.RopeMode.NEOX_FULL, prefill_state=state)
    torch.cuda.synchronize()
    assert st.key_cache_q8[:, :14].abs().sum().item() == 0 and st.key_cache_q8[:, 14:].abs().sum().item() > 0


def test_append_replay_is_deterministic(cuda):
    rng = np.random.default_rng(9)
    k, v = to_dev(ko.normal_f16(rng, (64, 1024))), to_dev(ko.normal_f16(rng, (64, 1024)))
    snaps = []
    for _ in range(4):
        st = kv.AttentionLayerKvCacheStorage(64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=8, head_dim=128, qblock=32)
        kv.launch_kv_store_quant(st.view(), k, v, None, 64, 0, rope_mode=kv.RopeMode.NEOX_FULL)
        snaps.append(torch.cat([st.key_cache_q8.flatten().view(torch.uint8), st.key_scales.flatten().view(torch.uint8)]).cpu())
    assert all(torch.equal(snaps[0], s) for s in snaps[1:])


def test_append_unaligned_inputs_bit_exact(cuda):
    # inputs that do not start on a 16-byte boundary take the element-wise loads: same bits
    rng = np.random.default_rng(12)
    T, H, d = 19, 8, 128
    k, v = ko.normal_f16(rng, (T, H * d)), ko.normal_f16(rng, (T, H * d))
    host = ko.HostCache(32, H, d, 32, 3)
    host.append(k.astype(np.float32), v.astype(np.float32), None, 3, rope_mode=1)
    st = device_storage_like(host)
    pad_k = torch.zeros(T * H * d + 8, dtype=torch.float16, device="cuda")
    pad_v = torch.zeros(T * H * d + 8, dtype=torch.float16, device="cuda")
    kd, vd = pad_k[1:1 + T * H * d].view(T, H * d), pad_v[3:3 + T * H * d].view(T, H * d)
    kd.copy_(to_dev(k)); vd.copy_(to_dev(v))
    assert kd.data_ptr() % 16 != 0 and vd.data_ptr() % 16 != 0
    kv.launch_kv_store_quant(st.view(), kd, vd, None, T, 3, rope_mode=kv.RopeMode.NEOX_FULL)
    torch.cuda.synchronize()
    assert_planes_equal(st, host, "unaligned inputs")
