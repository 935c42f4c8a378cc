"""Helpers shared by the GPU parity tests: move a host (oracle) cache to a device
storage object and back."""
import numpy as np
import torch

import kvoracle as ko
from miinfer_b200 import kv

PLANES = [("key_f16", "key_cache"), ("value_f16", "value_cache"), ("key_q8", "key_cache_q8"),
          ("key_scales", "key_scales"), ("value_q8", "value_cache_q8"), ("value_scales", "value_scales")]


def device_storage_like(host: ko.HostCache) -> kv.AttentionLayerKvCacheStorage:
    return kv.AttentionLayerKvCacheStorage(host.capacity, kv.KvCacheQuantMode(host.quant_mode), kv_heads=host.kv_heads,
                                           head_dim=host.head_dim, qblock=host.qblock)


def upload(host: ko.HostCache) -> kv.AttentionLayerKvCacheStorage:
    st = device_storage_like(host)
    for hname, dname in PLANES:
        h = getattr(host, hname)
        if h is None:
            continue
        t = getattr(st, dname)
        src = torch.from_numpy(h.view(np.int16) if h.dtype == np.uint16 else h)
        t.copy_(src.view(t.dtype) if t.dtype != src.dtype else src)
    return st


def plane_bits(st: kv.AttentionLayerKvCacheStorage, dname: str) -> np.ndarray:
    t = getattr(st, dname)
    if t.dtype == torch.float16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def assert_planes_equal(st: kv.AttentionLayerKvCacheStorage, host: ko.HostCache, what: str = "") -> None:
    for hname, dname in PLANES:
        h = getattr(host, hname)
        if h is None:
            assert getattr(st, dname) is None
            continue
        got = plane_bits(st, dname)
        if not np.array_equal(got, h):
            bad = np.argwhere(got != h)
            raise AssertionError(f"{what} plane {hname}: {len(bad)} of {h.size} elements differ, first at {bad[0]}: "
                                 f"gpu {got[tuple(bad[0])]} oracle {h[tuple(bad[0])]}")


def to_dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)
