"""GPU test of the C++ boundary: builds tests/shim_smoke.cpp against miinfer_shim.hpp + libb200kv.so and runs a
reference-style call sequence (store -> suffix attention -> decode attention) with the reference's own names."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def test_reference_named_launchers_through_the_shim(cuda, tmp_path):
    from miinfer_b200 import _lib

    exe = tmp_path / "shim_smoke"
    cmd = ["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{ROOT / 'include'}",
           f"-I{ROOT / 'miinfer_b200' / 'compat'}", str(ROOT / "tests" / "shim_smoke.cpp"), "-o", str(exe),
           str(_lib.LIB_PATH), "-Xlinker", f"-rpath={_lib.LIB_PATH.parent}"]
    subprocess.run(cmd, check=True, capture_output=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and "shim ok" in res.stdout, res.stdout + res.stderr
    assert "bytes=%d" % (2 * 96 * 4 * 258) in res.stdout     # the reference's raw_tokens_bytes formula, kv_cache.cpp:222
