"""GPU test of b200kv_decode_attn_static, the decode-attention entry point for callers that cannot allocate
device memory (a host that gave the whole device to its own memory pool, or a sandbox without allocation
calls): it must give the same result as b200kv_decode_attn with a caller-owned workspace, on two calls in a
row that share the library's built-in scratch array.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2.0e-3


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda):
    from miinfer_b200 import kv
    from miinfer_b200._lib import lib

    assert lib.b200kv_decode_static_scratch_bytes() == 8 << 20
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    H, Hq, d = 8, 32, 128
    ws = kv.decode_workspace(Hq, d)
    # two calls in a row with different caches, lengths and queries: the second must not see the first one's leftovers
    for call, (length, capacity) in enumerate(((3000, 3072), (777, 1024))):
        st = kv.AttentionLayerKvCacheStorage(capacity, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=d, qblock=32)
        k = torch.randn(length, H * d, generator=g, device="cuda").half()
        v = torch.randn(length, H * d, generator=g, device="cuda").half()
        kv.launch_kv_store_quant(st.view(), k, v, None, length, 0, rope_mode=kv.RopeMode.NEOX_FULL)
        q = torch.randn(Hq, d, generator=g, device="cuda").half()
        gate = torch.randn(Hq, d, generator=g, device="cuda")
        ref = torch.empty(Hq, d, device="cuda"); ref_g = torch.empty(Hq, d, device="cuda")
        kv.launch_decode_attention_quant(st.view(), q, query_heads=Hq, scale=d ** -0.5, cache_length=length, output=ref,
                                         gate=gate, gated_output=ref_g, workspace=ws)
        out = torch.full((Hq, d), float("nan"), device="cuda"); out_g = torch.full((Hq, d), float("nan"), device="cuda")
        view = st.view()
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200kv_decode_attn_static(C.byref(view), q.data_ptr(), 0, gate.data_ptr(), out.data_ptr(), out_g.data_ptr(),
                                           Hq, d ** -0.5, length, None, 0, stream)
        assert rc == 0, lib.b200kv_status_string(rc)
        torch.cuda.synchronize()
        assert np.max(np.abs((out - ref).cpu().numpy())) <= TOL, call
        assert np.max(np.abs((out_g - ref_g).cpu().numpy())) <= TOL, call
        assert torch.isfinite(out).all()
    # a shape whose scratch would not fit the fixed array is refused with a clear status, not truncated
    big = kv.AttentionLayerKvCacheStorage(64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=8, head_dim=256, qblock=32)
    bv = big.view()
    qb = torch.zeros(64, 256, device="cuda", dtype=torch.float16)
    ob = torch.zeros(64, 256, device="cuda")
    assert lib.b200kv_decode_workspace_bytes(64, 256, 1) > lib.b200kv_decode_static_scratch_bytes()
    assert lib.b200kv_decode_attn_static(C.byref(bv), qb.data_ptr(), 0, None, ob.data_ptr(), None, 64, 0.0625, 64, None, 0, None) == -5
