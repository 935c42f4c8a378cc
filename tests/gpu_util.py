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


def attention_error(got: np.ndarray, ref: np.ndarray):
    """(max-abs, relative L2) of an attention output against the oracle's."""
    diff = got.astype(np.float64) - ref.astype(np.float64)
    return float(np.max(np.abs(diff))), float(np.linalg.norm(diff) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30))


def assert_attention_close(got: np.ndarray, ref: np.ndarray, what: str, tol_abs: float = 2.0e-3, tol_rel: float = 1.0e-3):
    """Two gates: the absolute one the path's specification states (max-abs 2e-3 against the fp32-accumulated
    reference) and a relative one (relative L2), because at long contexts the outputs themselves are of the order
    of 1e-2 and the absolute gate alone would pass a visibly wrong result.  The measured errors are printed."""
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    max_abs, rel_l2 = attention_error(got, ref)
    print(f"[parity] {what}: max_abs {max_abs:.3e} rel_l2 {rel_l2:.3e} (output std {float(np.std(ref)):.3e})")
    assert max_abs <= tol_abs, f"{what}: max-abs error {max_abs:.3e} > {tol_abs}"
    assert rel_l2 <= tol_rel, f"{what}: relative L2 error {rel_l2:.3e} > {tol_rel}"
    return max_abs, rel_l2
