"""CPU tests of the host-side session code: prefix match outcomes (the reference's six failure modes,
experiments/EXP-V2-0014-prefix-state-reuse.md:34-39), file name, file format round trip and every rejection path
(corrupt header / hash / length / checksum, wrong model, quantization, quant mode, geometry) -- no GPU involved."""
import ctypes as C
import struct
from pathlib import Path

import numpy as np
import pytest

from miinfer_b200._lib import lib

HDR = C.c_char * 157


def arr(tokens):
    a = np.ascontiguousarray(tokens, np.uint32)
    return a, a.ctypes.data_as(C.c_void_p)


def test_prefix_match_outcomes_in_reference_order():
    cached, cp = arr([5, 6, 7, 8])
    def m(prompt, model=b"qwen", quant=b"Q4", version=20260925, clen=4, cmodel=b"qwen", cquant=b"Q4"):
        p, pp = arr(prompt)
        return lib.b200kv_prefix_match(cmodel, cquant, version, cp, clen, model, quant, pp, len(prompt))
    assert m([5, 6, 7, 8, 9]) == 0                      # ExactMatch
    assert m([5, 6, 0, 8, 9]) == 1                      # PrefixMismatch
    assert m([5, 6, 7, 8, 9], model=b"other") == 2      # ModelMismatch
    assert m([5, 6, 7, 8, 9], quant=b"Q8") == 3         # QuantizationMismatch
    assert m([5, 6, 7, 8, 9], clen=0) == 4              # EmptyCache
    assert m([5, 6, 7]) == 5                            # PromptShorterThanPrefix
    assert m([5, 6, 7, 8, 9], version=1) == 6           # VersionMismatch


def test_session_filename_format():
    buf = C.create_string_buffer(64)
    assert lib.b200kv_session_filename(0xABCDEF0123, 4096, buf, 64) == 0
    assert buf.value == b"sess_000000abcdef0123_p4096.miinfer"
    assert lib.b200kv_session_filename(1, 1, buf, 8) == -1


def write(path, tokens, payload, *, model=b"m", quant=b"q", layer_bytes=None, layers=2, geom=(8, 128, 32, 3)):
    t, tp = arr(tokens)
    lb = len(payload) // layers if layer_bytes is None else layer_bytes
    return lib.b200kv_session_write(str(path).encode(), model, quant, tp, len(tokens), payload.ctypes.data_as(C.c_void_p), lb, layers, *geom)


def read(path, *, model=b"m", quant=b"q", layers=2, geom=(8, 128, 32, 3), cap=1 << 20):
    toks = np.zeros(4096, np.uint32)
    out = np.zeros(cap, np.uint8)
    n = C.c_uint32()
    rc = lib.b200kv_session_read(str(path).encode(), model, quant, layers, *geom, toks.ctypes.data_as(C.c_void_p), toks.size, C.byref(n),
                                 out.ctypes.data_as(C.c_void_p), out.size)
    return rc, toks[:n.value], out


def test_session_file_round_trip_and_layout(tmp_path):
    rng = np.random.default_rng(3)
    tokens = [14990, 42, 31415, 2718, 7]
    payload = rng.integers(0, 256, 2 * 5 * 8 * 136 * 2, dtype=np.uint8)
    path = tmp_path / "sub" / "s.miinfer"
    assert write(path, tokens, payload) == 0 and path.exists() and not Path(str(path) + ".tmp").exists()
    raw = path.read_bytes()
    assert raw[:4] == b"MISS" and struct.unpack_from("<I", raw, 4)[0] == 20260928
    assert len(raw) == 157 + 4 * len(tokens) + payload.size + 48          # header | tokens | KV | trailer
    assert raw[157:157 + 20] == np.asarray(tokens, np.uint32).tobytes()
    hdr = HDR()
    toks = np.zeros(8, np.uint32)
    assert lib.b200kv_session_inspect(str(path).encode(), hdr, toks.ctypes.data_as(C.c_void_p), 8) == 0
    prefix_length, token_hash = struct.unpack_from("<IQ", hdr.raw, 104)
    assert prefix_length == 5 and token_hash == lib.b200kv_token_sequence_hash(arr(tokens)[0].ctypes.data_as(C.POINTER(C.c_uint32)), 5)
    gdn_layers, gdn_bytes, gqa_layers, mode, kv_bytes = struct.unpack_from("<IQIBQ", hdr.raw, 116)
    assert (gdn_layers, gdn_bytes, gqa_layers, mode, kv_bytes) == (0, 0, 2, 3, payload.size)
    rc, got_tokens, got = read(path)
    assert rc == 0 and list(got_tokens) == tokens and np.array_equal(got[:payload.size], payload)


def test_session_rejections(tmp_path):
    rng = np.random.default_rng(4)
    tokens = list(range(100, 140))
    payload = rng.integers(0, 256, 2 * 1000, dtype=np.uint8)
    path = tmp_path / "s.miinfer"
    assert write(path, tokens, payload) == 0
    good = path.read_bytes()
    assert read(path, model=b"other")[0] == -9 and read(path, quant=b"zz")[0] == -9          # valid file, someone else's
    assert read(path, layers=3)[0] == -9
    assert read(path, geom=(8, 128, 32, 1))[0] == -9      # kv quant mode: written by the reference, never checked by it
    assert read(path, geom=(8, 128, 128, 3))[0] == -9     # scale-block width
    assert read(path, geom=(4, 256, 32, 3))[0] == -9
    assert read(tmp_path / "missing.miinfer")[0] == -8

    def corrupt(offset, value=0xFF):
        b = bytearray(good)
        b[offset] ^= value
        p = tmp_path / "bad.miinfer"
        p.write_bytes(bytes(b))
        return read(p)[0]
    assert corrupt(0) == -7                      # magic
    assert corrupt(4) == -7                      # version
    assert corrupt(157 + 8) == -7                # a token: hash no longer matches
    assert corrupt(108) == -7                    # stored hash
    assert corrupt(157 + 160 + 17) == -7         # one payload byte: checksum
    assert corrupt(len(good) - 48) == -7         # trailer magic
    (tmp_path / "short.miinfer").write_bytes(good[:len(good) - 60])
    assert read(tmp_path / "short.miinfer")[0] == -7
    (tmp_path / "tiny.miinfer").write_bytes(good[:50])
    assert read(tmp_path / "tiny.miinfer")[0] == -7
    assert write(tmp_path / "e.miinfer", [], payload) == -1                  # empty prefix is refused
    assert write(tmp_path / "nodir" / "x" / "y.miinfer", tokens, payload) == 0    # parent directories are created


def test_find_longest_matching_session(tmp_path):
    payload = np.zeros(64, np.uint8)
    prompt = list(range(1, 50))
    assert write(tmp_path / "a.miinfer", prompt[:10], payload) == 0
    assert write(tmp_path / "b.miinfer", prompt[:30], payload) == 0
    assert write(tmp_path / "c.miinfer", prompt[:20] + [999], payload) == 0       # diverges
    assert write(tmp_path / "d.miinfer", prompt[:40], payload, model=b"other") == 0
    assert write(tmp_path / "e.miinfer", prompt + [1, 2], payload) == 0           # longer than the prompt
    (tmp_path / "junk.miinfer").write_bytes(b"not a session")
    p, pp = arr(prompt)
    out = C.create_string_buffer(512)
    n = C.c_uint32()
    assert lib.b200kv_session_find(str(tmp_path).encode(), b"m", b"q", pp, len(prompt), out, 512, C.byref(n)) == 0
    assert n.value == 30 and out.value.decode().endswith("b.miinfer")
    assert lib.b200kv_session_find(str(tmp_path).encode(), b"m", b"nope", pp, len(prompt), out, 512, C.byref(n)) == -9
    assert lib.b200kv_session_find(str(tmp_path / "absent").encode(), b"m", b"q", pp, len(prompt), out, 512, C.byref(n)) == -9
