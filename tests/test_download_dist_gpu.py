"""GPU tests of two host-facing helpers: the dequantising download of a cache side (the reference's
AttentionLayerKvCacheStorage::download_key / download_value, src/prefill_v2/kv_cache.cpp:132-212) and the C form of
the NCCL merge of sequence-sharded decode (b200kv_dist_*), here with a communicator of one rank -- the multi-rank
path runs in `bench.py --workload seqshard --exchange nccl-c --gpus N`."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_attention_close, to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,H,qb,mode", [(128, 8, 32, 3), (256, 4, 256, 3), (256, 4, 32, 1), (128, 2, 32, 0)])
def test_download_key_value_dequantise_like_the_reference(cuda, d, H, qb, mode):
    rng = np.random.default_rng(d + mode)
    L, cap = 37, 48
    host = ko.HostCache(cap, H, d, qb, mode)
    host.append(ko.normal_f16(rng, (L, H * d)).astype(np.float32), ko.normal_f16(rng, (L, H * d)).astype(np.float32), None, 0, rope_mode=1)
    st = upload(host)
    for side, got in (("key", st.download_key(L)), ("value", st.download_value(L))):
        q8 = getattr(host, f"{side}_q8")
        if q8 is not None:
            scales = ko.half_to_float(getattr(host, f"{side}_scales")[:, :L])                      # [H][L][d/qb]
            want = q8[:, :L].astype(np.float32).reshape(H, L, d // qb, qb) * scales[..., None]    # int8 value x the scale of its block
            want = want.reshape(H, L, d)
        else:
            want = ko.half_to_float(getattr(host, f"{side}_f16")[:, :L])
        assert got.shape == (H, L, d) and np.array_equal(got, want.astype(np.float32)), side
    with pytest.raises(RuntimeError):
        st.download_key(cap + 1)           # the reference throws (kv_cache.cpp:133-135)


def test_nccl_merge_from_c_with_a_communicator_of_one_rank(cuda):
    rng = np.random.default_rng(3)
    H, Hq, d, L = 4, 24, 256, 900          # a geometry the in-kernel exchange does not take (head_dim 256, 6 heads per kv head)
    host = ko.HostCache(1024, H, d, 32, 3)
    host.append(ko.normal_f16(rng, (L, H * d)).astype(np.float32), ko.normal_f16(rng, (L, H * d)).astype(np.float32), None, 0, rope_mode=0)
    st = upload(host)
    q16 = ko.normal_f16(rng, (Hq, d))
    gate = rng.standard_normal((Hq, d)).astype(np.float32)
    want, want_g = host.decode_ref(q16.astype(np.float32), d ** -0.5, L, gate)
    dm = kv.DistMerge(kv.DistMerge.unique_id(), 0, 1, Hq, d)
    try:
        ws = kv.decode_workspace(Hq, d)
        out = torch.full((Hq, d), float("nan"), device="cuda"); gated = torch.full((Hq, d), float("nan"), device="cuda")
        dm.decode_partials(st.view(), to_dev(q16), scale=d ** -0.5, range_begin=0, range_end=L, workspace=ws)
        dm.merge(output=out, gate=to_dev(gate), gated_output=gated)
        torch.cuda.synchronize()
    finally:
        dm.destroy()
    assert_attention_close(out.cpu().numpy(), want, "NCCL merge, one rank")
    assert_attention_close(gated.cpu().numpy(), want_g, "NCCL merge, one rank (gated)")
