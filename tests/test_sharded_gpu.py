"""Sequence-sharded decode with the cross-GPU merge inside the kernel (b200kv_decode_attn_sharded), on ONE GPU.
Two kernels that wait for each other must not run as separate launches on one device, so the second rank is
never launched here: its partial is computed beforehand with b200kv_decode_partials and written into the exchange
buffer as the tagged words a peer would have stored.  The real multi-process path (IPC-mapped buffers, NVLink
stores) is exercised by `bench.py --workload seqshard --gpus N`."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import to_dev, upload

pytestmark = pytest.mark.gpu
TOL = 2.0e-3
H, HQ, D = 8, 32, 128


def _tagged(values: torch.Tensor, phase: int) -> torch.Tensor:
    """fp32 values as the 8-byte words {value, tag = phase + 1} of the exchange format."""
    from miinfer_b200 import kv
    return kv.exchange_words(values, phase)


def _setup(n, seed):
    from miinfer_b200 import kv
    rng = np.random.default_rng(seed)
    host = ko.HostCache((n + 63) // 64 * 64, H, D, 32, 3)
    host.append(ko.normal_f16(rng, (n, H * D)).astype(np.float32), ko.normal_f16(rng, (n, H * D)).astype(np.float32), None, 0, rope_mode=0)
    q16 = ko.normal_f16(rng, (HQ, D))
    return kv, host, upload(host), q16, to_dev(q16)


def _reference(kv, st, q, n, ws):
    out = torch.empty(HQ, D, device="cuda")
    kv.launch_decode_attention_quant(st.view(), q, query_heads=HQ, scale=D ** -0.5, cache_length=n, output=out, workspace=ws)
    return out


def test_world_of_one_equals_plain_decode(cuda):
    kv, host, st, q16, q = _setup(3000, 11)
    ws = kv.decode_workspace(HQ, D)
    ref = _reference(kv, st, q, 3000, ws)
    from miinfer_b200._lib import lib
    words = lib.b200kv_exchange_bytes(HQ, D, 1) // 8
    buf = torch.zeros(words, dtype=torch.int64, device="cuda")
    ex = kv.Exchange.from_pointers([buf.data_ptr()], 0)
    for phase in (0, 1, 0):
        out = torch.full((HQ, D), float("nan"), device="cuda")
        kv.launch_decode_attention_sharded(st.view(), q, ex, query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=3000,
                                           phase=phase, output=out, workspace=ws)
        torch.cuda.synchronize()
        # world == 1 takes no exchange step at all: the buffer stays untouched
        assert float((out - ref).abs().max()) <= 1e-6
    assert int(buf.abs().sum()) == 0


@pytest.mark.parametrize("n,cut,phase", [(4096, 2048, 0), (5000, 1777, 1), (2500, 2500, 0), (4096, 1024, 36)])
def test_two_ranks_with_the_peer_partial_already_delivered(cuda, n, cut, phase):
    kv, host, st, q16, q = _setup(n, 23 + phase)
    ws = kv.decode_workspace(HQ, D)
    ref = _reference(kv, st, q, n, ws)
    # rank 1's shard [cut, n) reduced to one partial per head, the way its kernel would
    mine = kv.packed_partial(HQ, D, 1)
    pm, pl, pa = kv.partial_views(mine[0], HQ, D)
    kv.launch_decode_partials(st.view(), q, query_heads=HQ, scale=D ** -0.5, range_begin=cut, range_end=n,
                              part_m=pm, part_l=pl, part_acc=pa, workspace=ws)
    torch.cuda.synchronize()
    words_per_rank = HQ * (D + 2)
    own = torch.zeros(2 * 2 * words_per_rank, dtype=torch.int64, device="cuda")     # [phase][src rank][head][d + 2]
    peer = torch.zeros_like(own)                                                      # what rank 1 would receive
    slot_index = phase & 1      # the call number's lowest bit selects the slot, the number itself tags the words
    slot = own[(slot_index * 2 + 1) * words_per_rank:(slot_index * 2 + 2) * words_per_rank].view(HQ, D + 2)
    slot[:, :D] = _tagged(pa.view(HQ, D), phase)
    slot[:, D] = _tagged(pm, phase)
    slot[:, D + 1] = _tagged(pl, phase)
    ex = kv.Exchange.from_pointers([own.data_ptr(), peer.data_ptr()], 0)
    out = torch.full((HQ, D), float("nan"), device="cuda")
    gate = torch.randn(HQ, D, device="cuda")
    gated = torch.empty(HQ, D, device="cuda")
    kv.launch_decode_attention_sharded(st.view(), q, ex, query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=cut,
                                       phase=phase, output=out, gate=gate, gated_output=gated, workspace=ws)
    torch.cuda.synchronize()
    assert float((out - ref).abs().max()) <= 2e-5          # same partials, merged in a different order
    assert float((gated - ref * torch.sigmoid(gate)).abs().max()) <= 2e-5
    # against the CPU oracle as well
    want, _ = host.decode_ref(q16.astype(np.float32), D ** -0.5, n)
    assert np.max(np.abs(out.cpu().numpy() - want)) <= TOL
    # consumed words are zero again; rank 0's partial went to the peer's buffer, slot [phase][0], fully tagged
    assert int(own.abs().sum()) == 0
    sent = peer[(slot_index * 2) * words_per_rank:(slot_index * 2 + 1) * words_per_rank]
    assert bool(((sent >> 32) == phase + 1).all())
    other = torch.cat([peer[:(slot_index * 2) * words_per_rank], peer[(slot_index * 2 + 1) * words_per_rank:]])
    assert int(other.abs().sum()) == 0


@pytest.mark.parametrize("stale", [False, True])
def test_a_peer_that_never_delivers_poisons_the_output_and_sets_the_status_word(cuda, stale):
    """The wait for a peer is bounded: with nothing in the peer's slot -- or only the words of an EARLIER call,
    as a rank that arrives after its peers gave up would leave them -- the kernel gives up, writes NaN and
    reports the timeout in the registered status word.  After clearing, the next call works again."""
    kv, host, st, q16, q = _setup(1024, 5)
    ws = kv.decode_workspace(HQ, D)
    words_per_rank = HQ * (D + 2)
    own = torch.zeros(2 * 2 * words_per_rank, dtype=torch.int64, device="cuda")
    peer = torch.zeros_like(own)
    if stale:   # call 4's words sit in slot 0 where call 6 looks: same slot, other tag
        own[words_per_rank:2 * words_per_rank] = _tagged(torch.ones(words_per_rank, device="cuda"), 4)
    ex = kv.Exchange.from_pointers([own.data_ptr(), peer.data_ptr()], 0)
    out = torch.zeros(HQ, D, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kv.set_status_word(status)
    try:
        kv.launch_decode_attention_sharded(st.view(), q, ex, query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=1024,
                                           phase=6, output=out, workspace=ws)
        torch.cuda.synchronize()
        assert bool(torch.isnan(out).all())
        assert int(status.item()) & kv.STATUS_PEER_TIMEOUT
        # recovery as documented: zero the status word, clear the workspace and the exchange buffers, go on
        status.zero_(); own.zero_(); peer.zero_()
        kv.workspace_reset(ws)
        want = _reference(kv, st, q, 1024, ws)
        pm = torch.full((HQ,), float("-inf"), device="cuda"); pl = torch.zeros(HQ, device="cuda"); pa = torch.zeros(HQ, D, device="cuda")
        slot = own[(1 * 2 + 1) * words_per_rank:(1 * 2 + 2) * words_per_rank].view(HQ, D + 2)   # call 7 -> slot 1; the peer's shard is empty
        slot[:, :D] = _tagged(pa, 7); slot[:, D] = _tagged(pm, 7); slot[:, D + 1] = _tagged(pl, 7)
        kv.launch_decode_attention_sharded(st.view(), q, ex, query_heads=HQ, scale=D ** -0.5, range_begin=0, range_end=1024,
                                           phase=7, output=out, workspace=ws)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert float((out - want).abs().max()) <= 2e-5
    finally:
        kv.set_status_word(None)
