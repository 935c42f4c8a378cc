"""CPU tests of the C-ABI boundary: the library loads, exports every symbol
that include/b200kv.h declares, and rejects bad arguments without a GPU."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "b200kv.h").read_text()
    return sorted(set(re.findall(r"B200KV_API\s+[\w\s\*]+?\b(b200kv_\w+)\s*\(", text)))


def test_header_declarations_are_all_exported_and_bound():
    from miinfer_b200 import _lib

    names = declared_functions()
    assert len(names) >= 22
    raw = C.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in b200kv.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"


def test_header_compiles_as_plain_c(tmp_path):
    import subprocess

    src = tmp_path / "t.c"
    src.write_text('#include "b200kv.h"\nint main(void){ b200kv_view v; (void)v; return sizeof(b200kv_decode_state)==64 && sizeof(b200kv_prefill_state)==64 ? 0 : 1; }\n')
    exe = tmp_path / "t"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_version_status_strings_and_host_helpers():
    from miinfer_b200 import kv
    from miinfer_b200._lib import lib

    assert lib.b200kv_version() == 200
    assert lib.b200kv_status_string(0) == b"ok"
    assert b"workspace" in lib.b200kv_status_string(-5)
    # 136 B per 128-wide row for q8_0 blocks, (d+2) for the reference's row scale
    assert lib.b200kv_cache_bytes(1, 1, 128, 32, 3) == 2 * 136
    assert lib.b200kv_cache_bytes(10, 4, 256, 256, 3) == 2 * 10 * 4 * 258
    assert lib.b200kv_cache_bytes(10, 4, 256, 256, 0) == 2 * 10 * 4 * 512
    assert lib.b200kv_decode_workspace_bytes(32, 128, 1) == 3 * 128 * 32 * 130 * 4   # plain partials + twice that for tagged partials
    import kvoracle as ko

    toks = [14990, 42, 31415, 2718]
    assert kv.token_sequence_hash(toks) == ko.token_sequence_hash(toks)


def test_argument_errors_are_statuses_not_aborts():
    from miinfer_b200._lib import View, lib

    v = View()
    assert lib.b200kv_append(None, None, None, 0, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -1
    assert lib.b200kv_append(C.byref(v), None, None, 0, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -1  # capacity 0
    v = View(0, 0, 16, 16, 16, 16, 8, 2, 96, 32, 3)
    assert lib.b200kv_append(C.byref(v), 16, 16, 0, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -2   # head_dim 96
    v = View(0, 0, 16, 16, 16, 16, 8, 2, 128, 32, 3)
    assert lib.b200kv_append(C.byref(v), 16, 16, 0, None, 0, 1e6, 1e-6, 4, 6, None, None, None) == -6    # past capacity
    assert lib.b200kv_append(C.byref(v), 16, 16, 7, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -1    # dtype
    assert lib.b200kv_decode_attn(C.byref(v), 16, 0, None, None, None, None, 8, 0.1, 4, None, None, 0, 0, None) == -1  # no output
    assert lib.b200kv_decode_attn(C.byref(v), 16, 0, None, 16, None, None, 7, 0.1, 4, None, None, 0, 0, None) == -1   # 7 % 2
    assert lib.b200kv_decode_attn(C.byref(v), 16, 0, None, 16, None, None, 8, 0.1, 9, None, None, 0, 0, None) == -6   # length > capacity
    v = View(0, 0, 16, 16, 16, 24, 8, 2, 128, 32, 3)   # misaligned plane
    assert lib.b200kv_append(C.byref(v), 16, 16, 0, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -1
    assert lib.b200kv_snapshot_bytes(C.byref(View(0, 0, 16, 16, 16, 16, 8, 2, 128, 32, 3)), 5) == 2 * 5 * 2 * 136
    out = C.c_void_p()
    assert lib.b200kv_cache_create(C.byref(out), 0, 8, 128, 32, 3) == -1     # the reference ctor throws on capacity 0


def test_launch_without_gpu_fails_loudly():
    import torch
    from miinfer_b200._lib import View, lib

    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    v = View(0, 0, 16, 16, 16, 16, 8, 2, 128, 32, 3)
    assert lib.b200kv_append(C.byref(v), 16, 16, 0, None, 0, 1e6, 1e-6, 1, 0, None, None, None) == -4   # no device, no fallback
    assert lib.b200kv_prefill_prepare(C.byref(v), 4, 8, 16, 1 << 20, None) == -4
    assert lib.b200kv_prefill_attn_prepared(C.byref(v), 16, 0, None, 16, 4, 4, 8, 0.1, None, 16, 1 << 20, 4, None) == -4
    assert lib.b200kv_device_check(0) == -4
    # the batched-launch plan is host arithmetic and works anywhere; bad arguments are refused
    lengths = (C.c_uint32 * 3)(5000, 300, 9000)
    splits, bound = C.c_uint32(0), C.c_uint32(0)
    assert lib.b200kv_plan_batched_decode(lengths, 3, 8, 0, C.byref(splits), C.byref(bound)) == 0
    assert splits.value >= 1 and bound.value >= 9000
    assert lib.b200kv_plan_batched_decode(lengths, 3, 0, 0, C.byref(splits), C.byref(bound)) == -1
    assert lib.b200kv_plan_batched_decode(None, 3, 8, 0, C.byref(splits), C.byref(bound)) == -1
