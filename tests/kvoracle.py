"""ctypes binding of the CPU oracle (oracle/libkv_oracle.so) for the tests.

Test infrastructure only: the oracle is the checker, never the thing shipped.
Host-side caches are numpy arrays laid out exactly like the device planes.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
LIB = ORACLE_DIR / "libkv_oracle.so"


def build_oracle() -> None:
    src = ORACLE_DIR / "kv_oracle.c"
    if not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), str(LIB)], check=True, capture_output=True)


build_oracle()
_o = C.CDLL(str(LIB))


class HostView(C.Structure):
    _fields_ = [
        ("key_f16", C.c_void_p), ("value_f16", C.c_void_p),
        ("key_q8", C.c_void_p), ("key_scales", C.c_void_p),
        ("value_q8", C.c_void_p), ("value_scales", C.c_void_p),
        ("capacity", C.c_uint64), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("qblock", C.c_uint32), ("quant_mode", C.c_uint32),
    ]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


f32p = np.ctypeslib.ndpointer(np.float32, flags="C")
u32, u64, fl, i32, vp, sz = C.c_uint32, C.c_uint64, C.c_float, C.c_int, C.c_void_p, C.c_size_t
VP = C.POINTER(HostView)

_o.kvo_half_to_float.restype = fl
_o.kvo_half_to_float.argtypes = [C.c_uint16]
_o.kvo_float_to_half_rn.restype = C.c_uint16
_o.kvo_float_to_half_rn.argtypes = [fl]
_o.kvo_half_to_float_array.argtypes = [vp, vp, sz]
_o.kvo_float_to_half_array.argtypes = [vp, vp, sz]
_o.kvo_sincos_pinned.argtypes = [fl, C.POINTER(fl), C.POINTER(fl)]
_o.kvo_rope_heads.argtypes = [vp, vp, u32, u32, u32, fl, i32, i32]
_o.kvo_quantize_block.argtypes = [vp, u32, i32, vp, vp]
_o.kvo_append.restype = i32
_o.kvo_append.argtypes = [VP, vp, vp, vp, u32, u32, i32, fl, fl, i32, i32]
_o.kvo_decode_attn_ref.argtypes = [VP, vp, vp, vp, vp, u32, fl, u64]
_o.kvo_attention_splits_for_length.restype = u32
_o.kvo_attention_splits_for_length.argtypes = [u64]
_o.kvo_decode_partials.argtypes = [VP, vp, u32, fl, u64, u64, u32, vp, vp, vp]
_o.kvo_merge_partials.argtypes = [vp, vp, vp, u32, u32, u32, vp, vp, vp]
_o.kvo_decode_attn_splitk.argtypes = [VP, vp, vp, vp, vp, u32, fl, u64, u32]
_o.kvo_suffix_attn_ref.argtypes = [VP, vp, vp, vp, u32, u32, u32, fl]
_o.kvo_suffix_attn_splitk.argtypes = [VP, vp, vp, vp, u32, u32, u32, fl, u32]
_o.kvo_raw_tokens_bytes.restype = sz
_o.kvo_raw_tokens_bytes.argtypes = [VP, u64]
_o.kvo_download_raw.restype = i32
_o.kvo_download_raw.argtypes = [VP, u64, vp]
_o.kvo_upload_raw.restype = i32
_o.kvo_upload_raw.argtypes = [VP, u64, vp]
_o.kvo_token_sequence_hash.restype = u64
_o.kvo_token_sequence_hash.argtypes = [vp, sz]
_o.kvo_quantize_q8_1.argtypes = [vp, sz, vp]
_o.kvo_q_split_norm_rope.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, i32, fl, fl, i32]
_o.kvo_decode_state_advance.argtypes = [vp, vp, u32]
_o.kvo_num_threads.restype = i32
_o.kvo_set_num_threads.argtypes = [i32]

raw = _o


def set_threads(n: int) -> None:
    _o.kvo_set_num_threads(int(n))


def half_to_float(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, np.float32)
    _o.kvo_half_to_float_array(_p(bits), _p(out), bits.size)
    return out


def float_to_half(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    _o.kvo_float_to_half_array(_p(x), _p(out), x.size)
    return out


def sincos_pinned(angle: float):
    s, c = fl(), fl()
    _o.kvo_sincos_pinned(angle, C.byref(s), C.byref(c))
    return s.value, c.value


def rope_heads(x: np.ndarray, position: int, theta: float, rope_mode: int, trig_mode: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    heads, d = x.shape
    out = np.empty_like(x)
    _o.kvo_rope_heads(_p(x), _p(out), heads, d, position, theta, rope_mode, trig_mode)
    return out


def quantize_block(x: np.ndarray, quant_style: int = 0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.size, np.int8)
    s = np.zeros(1, np.uint16)
    _o.kvo_quantize_block(_p(x), x.size, quant_style, _p(q), _p(s))
    return q, int(s[0])


class HostCache:
    """numpy planes + a kvo_view over them (same layout as the device cache)."""

    def __init__(self, capacity, kv_heads, head_dim, qblock, quant_mode):
        self.capacity, self.kv_heads, self.head_dim = capacity, kv_heads, head_dim
        self.qblock, self.quant_mode = qblock, int(quant_mode)
        nblk = head_dim // qblock
        k_q8 = self.quant_mode in (1, 3)
        v_q8 = self.quant_mode in (2, 3)
        shape, sshape = (kv_heads, capacity, head_dim), (kv_heads, capacity, nblk)
        self.key_f16 = None if k_q8 else np.zeros(shape, np.uint16)
        self.value_f16 = None if v_q8 else np.zeros(shape, np.uint16)
        self.key_q8 = np.zeros(shape, np.int8) if k_q8 else None
        self.key_scales = np.zeros(sshape, np.uint16) if k_q8 else None
        self.value_q8 = np.zeros(shape, np.int8) if v_q8 else None
        self.value_scales = np.zeros(sshape, np.uint16) if v_q8 else None

    def view(self) -> HostView:
        return HostView(_p(self.key_f16), _p(self.value_f16), _p(self.key_q8), _p(self.key_scales),
                        _p(self.value_q8), _p(self.value_scales), self.capacity, self.kv_heads, self.head_dim,
                        self.qblock, self.quant_mode)

    def planes(self):
        return {n: getattr(self, n) for n in ("key_f16", "value_f16", "key_q8", "key_scales", "value_q8", "value_scales")
                if getattr(self, n) is not None}

    # -- oracle operations -----------------------------------------------------
    def append(self, key, value, k_norm_weight, base_position, *, rope_mode, theta=1.0e6, epsilon=1.0e-6,
               trig_mode=1, quant_style=0):
        key = np.ascontiguousarray(key, np.float32)
        value = np.ascontiguousarray(value, np.float32)
        w = None if k_norm_weight is None else np.ascontiguousarray(k_norm_weight, np.float32)
        v = self.view()
        rc = _o.kvo_append(C.byref(v), _p(key), _p(value), _p(w), key.shape[0], base_position, rope_mode, theta,
                           epsilon, trig_mode, quant_style)
        if rc != 0:
            raise ValueError("append outside the cache")

    def decode_ref(self, q, scale, length, gate=None):
        q = np.ascontiguousarray(q, np.float32)
        out = np.empty_like(q)
        gated = np.empty_like(q)
        g = None if gate is None else np.ascontiguousarray(gate, np.float32)
        v = self.view()
        _o.kvo_decode_attn_ref(C.byref(v), _p(q), _p(g), _p(out), _p(gated), q.shape[0], scale, length)
        return out, gated

    def decode_splitk(self, q, scale, length, num_splits=0, gate=None):
        q = np.ascontiguousarray(q, np.float32)
        out = np.empty_like(q)
        gated = np.empty_like(q)
        g = None if gate is None else np.ascontiguousarray(gate, np.float32)
        v = self.view()
        _o.kvo_decode_attn_splitk(C.byref(v), _p(q), _p(g), _p(out), _p(gated), q.shape[0], scale, length, num_splits)
        return out, gated

    def decode_partials(self, q, scale, begin, end, num_splits):
        q = np.ascontiguousarray(q, np.float32)
        hq, d = q.shape
        m = np.empty((num_splits, hq), np.float32)
        l = np.empty((num_splits, hq), np.float32)
        acc = np.empty((num_splits, hq, d), np.float32)
        v = self.view()
        _o.kvo_decode_partials(C.byref(v), _p(q), hq, scale, begin, end, num_splits, _p(m), _p(l), _p(acc))
        return m, l, acc

    def suffix_ref(self, q, gate, base_position, scale):
        q = np.ascontiguousarray(q, np.float32)
        t, hq, d = q.shape
        out = np.zeros_like(q)
        g = None if gate is None else np.ascontiguousarray(gate, np.float32)
        v = self.view()
        _o.kvo_suffix_attn_ref(C.byref(v), _p(q), _p(g), _p(out), t, base_position, hq, scale)
        return out

    def suffix_splitk(self, q, gate, base_position, scale, num_splits=32):
        q = np.ascontiguousarray(q, np.float32)
        t, hq, d = q.shape
        out = np.zeros_like(q)
        g = None if gate is None else np.ascontiguousarray(gate, np.float32)
        v = self.view()
        _o.kvo_suffix_attn_splitk(C.byref(v), _p(q), _p(g), _p(out), t, base_position, hq, scale, num_splits)
        return out

    def raw_tokens_bytes(self, tokens):
        v = self.view()
        return int(_o.kvo_raw_tokens_bytes(C.byref(v), tokens))

    def download_raw(self, tokens):
        blob = np.zeros(self.raw_tokens_bytes(tokens), np.uint8)
        v = self.view()
        assert _o.kvo_download_raw(C.byref(v), tokens, _p(blob)) == 0
        return blob

    def upload_raw(self, blob, tokens):
        blob = np.ascontiguousarray(blob, np.uint8)
        v = self.view()
        assert _o.kvo_upload_raw(C.byref(v), tokens, _p(blob)) == 0


def merge_partials(m, l, acc, gate=None):
    m, l, acc = (np.ascontiguousarray(a, np.float32) for a in (m, l, acc))
    parts, hq, d = acc.shape
    out = np.empty((hq, d), np.float32)
    gated = np.empty((hq, d), np.float32)
    g = None if gate is None else np.ascontiguousarray(gate, np.float32)
    _o.kvo_merge_partials(_p(m), _p(l), _p(acc), parts, hq, d, _p(g), _p(out), _p(gated))
    return out, gated


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    """Q8_1 blocks (36 bytes each) of an fp32 array whose size is a multiple of 32."""
    x = np.ascontiguousarray(x, np.float32)
    blocks = np.zeros((x.size // 32, 36), np.uint8)
    _o.kvo_quantize_q8_1(_p(x), x.size, _p(blocks))
    return blocks


def q_split_norm_rope(qfull: np.ndarray, weight, base_position: int, *, rope_mode: int, theta=1.0e6, epsilon=1.0e-6, trig_mode=1):
    """qfull fp32 [token][heads][2*d] -> (query [token][heads][d], gate [token][heads][d])."""
    qfull = np.ascontiguousarray(qfull, np.float32)
    t, h, d2 = qfull.shape
    d = d2 // 2
    q = np.empty((t, h, d), np.float32)
    g = np.empty((t, h, d), np.float32)
    w = None if weight is None else np.ascontiguousarray(weight, np.float32)
    _o.kvo_q_split_norm_rope(_p(qfull), _p(w), _p(q), _p(g), t, base_position, h, d, rope_mode, theta, epsilon, trig_mode)
    return q, g


def decode_state_advance(state: np.ndarray, token_output: np.ndarray) -> None:
    assert state.dtype == np.uint32 and token_output.dtype == np.uint32
    _o.kvo_decode_state_advance(_p(state), _p(token_output), token_output.size)


def token_sequence_hash(tokens) -> int:
    a = np.ascontiguousarray(tokens, np.uint32)
    return int(_o.kvo_token_sequence_hash(_p(a), a.size))


# -- seeded synthetic inputs (fp16 N(0,1) activations, as the benchmark workloads use) ----------
class StdNormalStream:
    """std::mt19937(seed) feeding std::normal_distribution<float>(mean, stddev), drawn by the C++ standard library itself
    (oracle/std_stream.cpp): the stream a C++ test sees."""

    def __init__(self, seed: int, mean: float, stddev: float):
        lib_path = ORACLE_DIR / "libstd_stream.so"
        src = ORACLE_DIR / "std_stream.cpp"
        if not lib_path.exists() or lib_path.stat().st_mtime < src.stat().st_mtime:
            subprocess.run(["make", "-C", str(ORACLE_DIR), str(lib_path)], check=True, capture_output=True)
        self._lib = C.CDLL(str(lib_path))
        self._lib.std_stream_new.restype = C.c_void_p
        self._lib.std_stream_new.argtypes = [C.c_uint, C.c_float, C.c_float]
        self._lib.std_stream_fill.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        self._lib.std_stream_free.argtypes = [C.c_void_p]
        self._s = self._lib.std_stream_new(seed, mean, stddev)

    def draw(self, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        self._lib.std_stream_fill(self._s, _p(out), count)
        return out

    def __del__(self):
        if getattr(self, "_s", None):
            self._lib.std_stream_free(self._s)
            self._s = None


def normal_f16(rng: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    """fp16 N(0, std) values as a float16 array (exactly representable inputs)."""
    return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float16)
