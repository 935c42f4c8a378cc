"""GPU tests of the in-VRAM snapshot pool and of prefix reuse around real layer caches: a session restored from
the pool (or from a session file chosen by the reuse policy) must decode bit-identically to the session the
snapshot was taken from -- the reference's gate for prefix reuse (token-for-token parity cold vs restored,
bench/v2_0028_persistent_session_bench.cpp:235-257)."""
import numpy as np
import pytest
import torch

import kvoracle as ko
from gpu_util import assert_planes_equal, to_dev, upload
from miinfer_b200 import kv

pytestmark = pytest.mark.gpu
H, HQ, D, LAYERS = 8, 32, 128, 3


def _session(rng, tokens):
    hosts = []
    for _ in range(LAYERS):
        h = ko.HostCache(tokens + 64, H, D, 32, 3)
        h.append(ko.normal_f16(rng, (tokens, H * D)).astype(np.float32), ko.normal_f16(rng, (tokens, H * D)).astype(np.float32), None, 0, rope_mode=1)
        hosts.append(h)
    return hosts, [upload(h) for h in hosts]


def _decode_all(sts, q, length):
    ws = kv.decode_workspace(HQ, D)
    outs = []
    for st in sts:
        o = torch.empty(HQ, D, device="cuda")
        kv.launch_decode_attention_quant(st.view(), q, query_heads=HQ, scale=D ** -0.5, cache_length=length, output=o, workspace=ws)
        outs.append(o)
    torch.cuda.synchronize()
    return outs


def test_restore_from_the_pool_decodes_bit_identically(cuda):
    rng = np.random.default_rng(31)
    P = 1024
    hosts, sts = _session(rng, P)
    tokens = [int(t) for t in rng.integers(0, 150000, P)]
    pool = kv.SnapshotPool("qwen3-8b", "q4_0", granularity=512)
    assert pool.capture(tokens, sts)
    assert pool.capture(tokens[:512], sts)            # a shorter snapshot of the same conversation
    st = pool.stats()
    assert st["entries"] == 2 and st["bytes"] >= LAYERS * (P + 512) * H * 136 * 2
    fresh = [kv.AttentionLayerKvCacheStorage(P + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=D, qblock=32) for _ in range(LAYERS)]
    assert pool.restore(tokens + [1, 2, 3], fresh) == P           # longest proper prefix
    q = to_dev(ko.normal_f16(rng, (HQ, D)))
    for a, b in zip(_decode_all(sts, q, P), _decode_all(fresh, q, P)):
        assert torch.equal(a, b)
    short = [kv.AttentionLayerKvCacheStorage(P + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=D, qblock=32) for _ in range(LAYERS)]
    assert pool.restore(tokens[:700], short) == 512
    for a, b in zip(_decode_all(sts, q, 512), _decode_all(short, q, 512)):
        assert torch.equal(a, b)
    assert pool.restore([9, 9, 9], short) == 0
    # caches of another shape are refused, not overwritten
    other = [kv.AttentionLayerKvCacheStorage(P + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=4, head_dim=256, qblock=32) for _ in range(LAYERS)]
    with pytest.raises(kv.B200KvError):
        pool.restore(tokens + [1], other)
    # eviction frees device memory and the evicted prefix is gone
    small = kv.SnapshotPool("qwen3-8b", "q4_0", max_entries=1, granularity=512)
    assert small.capture(tokens[:512], sts) and small.capture(tokens, sts)
    assert small.stats()["entries"] == 1 and small.stats()["evictions"] == 1
    assert small.restore(tokens[:600], short) == 0 and small.restore(tokens + [4], short) == P


def test_reuse_policy_around_real_caches_resident_pool_and_disk(cuda, tmp_path):
    rng = np.random.default_rng(32)
    P = 768
    hosts, sts = _session(rng, P)
    prompt = [int(t) for t in rng.integers(0, 150000, P + 40)]
    pool = kv.SnapshotPool("qwen3-8b", "q4_0", granularity=256)
    ctx = kv.ReusableContext("qwen3-8b", "q4_0", sts, pool=pool, cache_prefix_len=P, persistent_session_dir=str(tmp_path))
    assert not ctx.begin(prompt)["reuse_hit"]
    done = ctx.commit(prompt)                         # as after the first prefill: the prefix is cached, pooled and written to disk
    assert done == {"cached_length": P, "wrote_file": True}
    assert ctx.commit(prompt)["wrote_file"] is False  # the file exists: not written again
    assert ctx.begin(prompt)["source"] == 1           # resident
    q = to_dev(ko.normal_f16(rng, (HQ, D)))
    want = _decode_all(sts, q, P)
    # a second set of caches (another request slot of the same model): served by the pool
    slot2 = [kv.AttentionLayerKvCacheStorage(P + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=D, qblock=32) for _ in range(LAYERS)]
    ctx2 = kv.ReusableContext("qwen3-8b", "q4_0", slot2, pool=pool, persistent_session_dir=str(tmp_path))
    hit = ctx2.begin(prompt)
    assert hit["reuse_hit"] and hit["source"] == 2 and hit["prefix_tokens_reused"] == P and hit["suffix_tokens_dispatched"] == 40 and hit["restore_ms"] > 0
    for a, b in zip(want, _decode_all(slot2, q, P)):
        assert torch.equal(a, b)
    # a third set with no pool (a fresh process): served by the session directory
    slot3 = [kv.AttentionLayerKvCacheStorage(P + 64, kv.KvCacheQuantMode.kQ8Q8, kv_heads=H, head_dim=D, qblock=32) for _ in range(LAYERS)]
    hit3 = kv.ReusableContext("qwen3-8b", "q4_0", slot3, persistent_session_dir=str(tmp_path)).begin(prompt)
    assert hit3["reuse_hit"] and hit3["source"] == 3 and hit3["prefix_tokens_reused"] == P
    for a, b in zip(want, _decode_all(slot3, q, P)):
        assert torch.equal(a, b)
    for st, h in zip(slot3, hosts):
        restored = ko.HostCache(P + 64, H, D, 32, 3)
        for name in ("key_q8", "value_q8", "key_scales", "value_scales"):
            getattr(restored, name)[:, :P] = getattr(h, name)[:, :P]
        assert_planes_equal(st, restored, "restored from the session directory")
