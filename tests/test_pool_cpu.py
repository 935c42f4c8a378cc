"""CPU tests of the snapshot pool's index and eviction and of the prefix-reuse policy (host logic only: entries are
captured without a payload and the policy runs with no layer caches, so no device is touched).  The behaviour
asserted is that of MIInfer's session checkpoints (tools/miinfer_cli.cpp:1043-1228) and of the reuse branch of
PrefillV2Model::generate (src/prefill_v2/model.cpp:751-775, 868-887)."""
import ctypes as C

import numpy as np

from miinfer_b200 import kv
from miinfer_b200._lib import lib


def seq(n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, 150000, n)]


def test_longest_proper_prefix_lookup_in_the_radix_index():
    pool = kv.SnapshotPool("m", "q", granularity=512)
    base = seq(2048)
    assert pool.capture(base[:512], index_only_bytes=10)
    assert pool.capture(base[:1536], index_only_bytes=10)
    other = base[:700] + seq(324, 1)          # shares 700 tokens, then parts inside an edge
    assert pool.capture(other, index_only_bytes=10)
    assert pool.lookup(base) == (1536, 1536)
    assert pool.lookup(base[:1536]) == (512, 1536)      # a snapshot as long as the prompt cannot serve it: one token must still run
    assert pool.lookup(base[:512]) == (0, 512)
    assert pool.lookup(base[:100]) == (0, 100)
    assert pool.lookup(other + [5]) == (1024, 1024)
    assert pool.lookup(base[:700] + [1, 2, 3]) == (512, 700)
    assert pool.lookup(seq(50, 9)) == (0, 0)
    # another model or weight quantization finds nothing
    assert pool.lookup(base, model_id="other") == (0, 0)
    assert pool.lookup(base, quantization="q8") == (0, 0)
    st = pool.stats()
    assert st["entries"] == 3 and st["hits"] == 4 and st["captures"] == 3


def test_capture_granularity_budget_and_least_recently_used_eviction():
    pool = kv.SnapshotPool("m", "q", max_entries=3, max_bytes=1000, granularity=512)
    a, b, c, d = (seq(512, s) for s in (1, 2, 3, 4))
    assert not pool.capture(a[:100], index_only_bytes=1)       # not a multiple of the prefill tile
    assert not pool.capture([], index_only_bytes=1)
    assert not pool.capture(a, index_only_bytes=2000)          # larger than the whole budget
    assert pool.capture(a, index_only_bytes=300) and pool.capture(b, index_only_bytes=300) and pool.capture(c, index_only_bytes=300)
    assert pool.lookup(a + [1])[0] == 512                      # touch a: b is now the oldest
    assert pool.capture(d, index_only_bytes=300)               # entry limit: evicts b
    assert pool.lookup(b + [1])[0] == 0 and pool.lookup(a + [1])[0] == 512 and pool.lookup(c + [1])[0] == 512
    big = seq(1024, 5)
    assert pool.capture(big, index_only_bytes=700)             # byte budget: evicts until 700 more fit
    st = pool.stats()
    assert st["bytes"] <= 1000 and st["entries"] == 2 and pool.lookup(big + [1])[0] == 1024
    assert pool.capture(big, index_only_bytes=700) and pool.stats()["entries"] == 2     # same tokens: refreshed, not duplicated
    assert st["skipped"] == 3


def test_reuse_policy_resident_prefix_then_pool_then_nothing():
    prompt = seq(1500)
    pool = kv.SnapshotPool("qwen", "q4_k_m", granularity=512)
    ctx = kv.ReusableContext("qwen", "q4_k_m", None, pool=pool, cache_prefix_len=1024)
    first = ctx.begin(prompt)
    assert not first["reuse_hit"] and first["suffix_tokens_dispatched"] == 1500 and first["prefix_tokens_reused"] == 0
    assert ctx.commit(prompt) == {"cached_length": 1024, "wrote_file": False}       # first 1024 tokens are now resident and pooled
    # same prompt again: the resident prefix serves it, nothing is copied
    again = ctx.begin(prompt)
    assert again["reuse_hit"] and again["source"] == 1 and again["prefix_tokens_reused"] == 1024 and again["suffix_tokens_dispatched"] == 476
    assert again["gqa_kv_reused_tokens"] == 1024
    # a prompt that only equals the cached prefix cannot reuse it (the last token's logits need a forward pass)
    assert not ctx.begin(prompt[:1024])["reuse_hit"]
    # that call invalidated the resident prefix (the caches are refilled from 0); the pool still has the snapshot
    from_pool = ctx.begin(prompt)
    assert from_pool["reuse_hit"] and from_pool["source"] == 2 and from_pool["prefix_tokens_reused"] == 1024
    # another conversation: miss
    assert not ctx.begin(seq(900, 3))["reuse_hit"]
    # reuse switched off
    off = kv.ReusableContext("qwen", "q4_k_m", None, pool=pool, enable_prefix_reuse=False)
    off.resident_tokens = prompt[:1024]
    assert not off.begin(prompt)["reuse_hit"]


def test_reuse_policy_finds_a_session_file_and_insists_on_a_proper_prefix(tmp_path):
    tokens = seq(600, 11)
    H, d, layers = 2, 128, 2
    layer_bytes = 2 * 300 * H * (d + 2 * (d // 32))
    payload = np.zeros(layers * layer_bytes, np.uint8)
    name = f"sess_{kv.token_sequence_hash(tokens[:300]):016x}_p300.miinfer"
    toks = (C.c_uint32 * 300)(*tokens[:300])
    assert lib.b200kv_session_write(str(tmp_path / name).encode(), b"qwen", b"q4", toks, 300, payload.ctypes.data, layer_bytes, layers, H, d, 32, 3) == 0
    ctx = kv.ReusableContext("qwen", "q4", None, persistent_session_dir=str(tmp_path))
    hit = ctx.begin(tokens)
    assert hit["reuse_hit"] and hit["source"] == 3 and hit["prefix_tokens_reused"] == 300 and hit["suffix_tokens_dispatched"] == 300
    assert not kv.ReusableContext("qwen", "q4", None, persistent_session_dir=str(tmp_path)).begin(tokens[:300])["reuse_hit"]
    assert not kv.ReusableContext("other", "q4", None, persistent_session_dir=str(tmp_path)).begin(tokens)["reuse_hit"]
