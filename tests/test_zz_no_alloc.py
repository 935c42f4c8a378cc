"""GPU test of b200kv_decode_attn_static, the decode-attention entry point for callers that cannot allocate
device memory (a host that gave the whole device to its own memory pool, or a sandbox without allocation
calls): it must give the same result as b200kv_decode_attn with a caller-owned workspace -- the two run the
same kernels with the same split count, so the results must be bit-equal -- and agree with the CPU oracle, on
calls in a row that share the library's built-in scratch array, without the amount of free device memory
changing.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda):
    from miinfer_b200 import kv
    from miinfer_b200._lib import lib

    assert lib.b200kv_decode_static_scratch_bytes() == 8 << 20
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    # calls in a row with different caches, lengths and queries: a call must not see the previous one's leftovers
    import kvoracle as ko
    from gpu_util import assert_attention_close, upload

    rng = np.random.default_rng(99)
    # (length, capacity, cache mode, kv heads, query heads, head_dim, split count): streaming kernel twice, then the generic one
    cases = ((3000, 3072, 3, 8, 32, 128, 0), (777, 1024, 3, 8, 32, 128, 5), (300, 304, 1, 4, 8, 256, 0))
    free_before = None
    for call, (length, capacity, mode, H, Hq, d, splits) in enumerate(cases):
        host = ko.HostCache(capacity, H, d, 32, mode)
        host.append(ko.normal_f16(rng, (length, H * d)).astype(np.float32), ko.normal_f16(rng, (length, H * d)).astype(np.float32),
                    None, 0, rope_mode=1)
        st = upload(host)
        q16 = ko.normal_f16(rng, (Hq, d))
        q = torch.from_numpy(q16).cuda()
        gate = torch.randn(Hq, d, generator=g, device="cuda")
        ws = kv.decode_workspace(Hq, d)
        ref = torch.empty(Hq, d, device="cuda"); ref_g = torch.empty(Hq, d, device="cuda")
        kv.launch_decode_attention_quant(st.view(), q, query_heads=Hq, scale=d ** -0.5, cache_length=length, output=ref,
                                         gate=gate, gated_output=ref_g, workspace=ws, num_splits=splits)
        out = torch.full((Hq, d), float("nan"), device="cuda"); out_g = torch.full((Hq, d), float("nan"), device="cuda")
        state = kv.make_decode_state(length - 1)
        view = st.view()
        stream = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        if call > 0:
            free_before = torch.cuda.mem_get_info()[0]     # the first call may still load the kernels' module
        # odd calls take the length from device state (position + 1), as a replayed graph would
        rc = lib.b200kv_decode_attn_static(C.byref(view), q.data_ptr(), 0, gate.data_ptr(), out.data_ptr(), out_g.data_ptr(),
                                           Hq, d ** -0.5, 0 if call % 2 else length, state.data_ptr() if call % 2 else None, splits, stream)
        assert rc == 0, lib.b200kv_status_string(rc)
        torch.cuda.synchronize()
        if free_before is not None:
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point must not allocate device memory"
        if call % 2 == 0:   # same kernels, same split count, same reduction order: bit-equal
            assert torch.equal(out, ref) and torch.equal(out_g, ref_g), call
        else:               # the device-side length sizes the launch for the whole capacity: another split count
            assert float((out - ref).abs().max()) <= 2e-5, call
        want, want_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, length, gate.cpu().numpy())
        assert_attention_close(out.cpu().numpy(), want, f"static entry point, call {call}")
        assert_attention_close(out_g.cpu().numpy(), want_g, f"static entry point (gated), call {call}")
    # a shape whose scratch would not fit the fixed array is refused with a clear status, not truncated
    big = kv.AttentionLayerKvCacheStorage(64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=8, head_dim=256, qblock=32)
    bv = big.view()
    qb = torch.zeros(64, 256, device="cuda", dtype=torch.float16)
    ob = torch.zeros(64, 256, device="cuda")
    assert lib.b200kv_decode_workspace_bytes(64, 256, 1) > lib.b200kv_decode_static_scratch_bytes()
    assert lib.b200kv_decode_attn_static(C.byref(bv), qb.data_ptr(), 0, None, ob.data_ptr(), None, 64, 0.0625, 64, None, 0, None) == -5
