"""Generates the committed golden fixtures.  Run in a container that holds the
MIInfer source tree (--ref PATH, or the MIINFER_REF environment variable); the tests only read the .npz files.

  python tests/golden/make_golden.py --ref PATH_TO_MIINFER

1. m4a4_four_position.npz -- the reference's own stored layer-0 traces for the
   KV path (tests/reference/qwen3/m4a4-four-position/, README there lists the
   checkpoints): per position P in 0..3 the tensors q_normed(6) q_rope(7)
   k_normed(13) k_rope(14) attention_output(19) and the cache-k / cache-v write
   vectors.  Shapes: q 32x128, k/v 8x128.  These are the known-answer vectors the
   reference's tests/qwen3_kv_cache_test.cpp checks with tolerances 2.5e-2 (RoPE)
   and 2.0e-2 (attention).
2. m4b_layers.npz -- single-position RoPE/attention traces of deeper layers
   (tests/reference/qwen3/m4b-layer6, m4b-layer35).
3. ref_host_primitives.npz -- outputs of the reference's OWN host primitives
   (oracle/_ref/libmiinfer_host_ref.so = src/qwen3_primitives.cpp compiled in
   place) on seeded inputs: fp16_bits_to_float over all 65536 patterns,
   rope_qwen3_reference, softmax_reference, rms_norm_reference.
"""
from __future__ import annotations

import argparse
import os
import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def load_f32(path: Path, shape):
    a = np.fromfile(path, dtype="<f4")
    assert a.size == int(np.prod(shape)), (path, a.size, shape)
    return a.reshape(shape)


def four_position(ref: Path) -> None:
    d = ref / "tests/reference/qwen3/m4a4-four-position"
    out = {}
    for p in range(4):
        out[f"q_normed_{p}"] = load_f32(d / f"pos-{p}-6.f32", (32, 128))
        out[f"q_rope_{p}"] = load_f32(d / f"pos-{p}-7.f32", (32, 128))
        out[f"k_normed_{p}"] = load_f32(d / f"pos-{p}-13.f32", (8, 128))
        out[f"k_rope_{p}"] = load_f32(d / f"pos-{p}-14.f32", (8, 128))
        out[f"attention_output_{p}"] = load_f32(d / f"pos-{p}-19.f32", (32, 128))
        out[f"cache_k_{p}"] = load_f32(d / f"pos-{p}-cache-k.f32", (8, 128))
        out[f"cache_v_{p}"] = load_f32(d / f"pos-{p}-cache-v.f32", (8, 128))
    np.savez_compressed(HERE / "m4a4_four_position.npz", **out)


def deeper_layers(ref: Path) -> None:
    out = {}
    for layer in (6, 35):
        d = ref / f"tests/reference/qwen3/m4b-layer{layer}"
        out[f"q_normed_{layer}"] = load_f32(d / "q-normed.f32", (32, 128))
        out[f"q_rope_{layer}"] = load_f32(d / "q-rope.f32", (32, 128))
        out[f"k_normed_{layer}"] = load_f32(d / "k-normed.f32", (8, 128))
        out[f"k_rope_{layer}"] = load_f32(d / "k-rope.f32", (8, 128))
        v_file = d / "v-reshape.f32"
        if not v_file.exists():
            v_file = d / "v-projection.f32"  # same 1024 values before the [8][128] reshape
        out[f"v_reshape_{layer}"] = load_f32(v_file, (8, 128))
        out[f"attention_output_{layer}"] = load_f32(d / "attention-output.f32", (32, 128))
    np.savez_compressed(HERE / "m4b_layers.npz", **out)


def host_primitives() -> None:
    lib = C.CDLL(str(ROOT / "oracle/_ref/libmiinfer_host_ref.so"))
    lib.ref_fp16_bits_to_float.restype = C.c_float
    lib.ref_fp16_bits_to_float.argtypes = [C.c_uint16]
    vp, sz, fl = C.c_void_p, C.c_size_t, C.c_float
    lib.ref_rope_qwen3.argtypes = [vp, vp, sz, sz, sz, fl]
    lib.ref_softmax.argtypes = [vp, vp, sz]
    lib.ref_rms_norm.argtypes = [vp, vp, vp, sz, fl]
    ptr = lambda a: a.ctypes.data_as(vp)
    rng = np.random.default_rng(42)
    out = {}
    out["fp16_all"] = np.array([lib.ref_fp16_bits_to_float(b) for b in range(65536)], np.float32)
    for d, heads in ((128, 8), (256, 4)):
        x = rng.standard_normal((heads, d), dtype=np.float32)
        out[f"rope_in_{d}"] = x
        for pos in (0, 1, 7, 1000, 32767, 131071):
            y = np.empty_like(x)
            assert lib.ref_rope_qwen3(ptr(x), ptr(y), heads, d, pos, 1.0e6) == 0
            out[f"rope_out_{d}_{pos}"] = y
    for n in (1, 5, 4097):
        s = (rng.standard_normal(n, dtype=np.float32) * 3).astype(np.float32)
        y = np.empty_like(s)
        assert lib.ref_softmax(ptr(s), ptr(y), n) == 0
        out[f"softmax_in_{n}"], out[f"softmax_out_{n}"] = s, y
    x = rng.standard_normal(256, dtype=np.float32)
    w = rng.standard_normal(256, dtype=np.float32)
    y = np.empty_like(x)
    assert lib.ref_rms_norm(ptr(x), ptr(w), ptr(y), 256, 1.0e-6) == 0
    out["rms_in"], out["rms_w"], out["rms_out"] = x, w, y
    np.savez_compressed(HERE / "ref_host_primitives.npz", **out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("MIINFER_REF"), required=os.environ.get("MIINFER_REF") is None,
                    help="root of the MIInfer source tree")
    args = ap.parse_args()
    four_position(Path(args.ref))
    deeper_layers(Path(args.ref))
    host_primitives()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
