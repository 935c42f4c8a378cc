"""Writes tests/golden/quant_kv_attention_pin.json: the error figures of MIInfer's quantized-attention test recipe
(tests/qwen3_quant_kv_attention_test.cpp:79-154), computed by the CPU oracle on the very inputs that test draws.

The recipe: std::mt19937(42) and std::normal_distribution<float>(0, 0.5); 24 query heads, 4 kv heads, head_dim 256,
scale 1/16; four cases (prefix, suffix) = (64, 16), (512, 64), (4096, 128), (16384, 512) drawn one after the other from
the same stream -- q, gate, then per kv head and position a K vector and a V vector; K and V quantised per row by the
test's host quantiser (amax / 127, round half away, clamp +-127, fp16 scale); suffix attention with a sigmoid gate in
four cache modes; errors of the three quantised modes against the fp16 one.  The oracle's kernel-order restatement of
the reference's split-K suffix kernel (32 splits, as the test asks for) stands in for the GPU kernels.

Usage: python tests/golden/make_statistical_pin.py [--cases 4]   (the fourth case takes a few minutes of CPU)
"""
import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import kvoracle as ko  # noqa: E402

CASES = [(64, 16), (512, 64), (4096, 128), (16384, 512)]
HQ, HKV, D = 24, 4, 256
SCALE = 1.0 / 16.0


def metrics(ref: np.ndarray, test: np.ndarray) -> dict:
    r = ref.astype(np.float64).ravel()
    t = test.astype(np.float64).ravel()
    d = np.abs(r - t)
    return {"max_abs": float(d.max()), "mae": float(d.mean()), "rmse": float(np.sqrt((d * d).mean())),
            "cos": float(r @ t / (np.sqrt(r @ r) * np.sqrt(t @ t) + 1e-12))}


def draw_cases(count: int):
    """Inputs of the first `count` cases in order (the stream runs on from one case into the next):
    (prefix, suffix, q [T][24][256], gate, k [P + T][4 * 256], v)."""
    stream = ko.StdNormalStream(42, 0.0, 0.5)
    for prefix, suffix in CASES[:count]:
        total = prefix + suffix
        q = stream.draw(suffix * HQ * D).reshape(suffix, HQ, D)
        gate = stream.draw(suffix * HQ * D).reshape(suffix, HQ, D)
        kv = stream.draw(HKV * total * 2 * D).reshape(HKV, total, 2, D)   # per head and position: K vector, then V vector
        k = np.ascontiguousarray(kv[:, :, 0, :].transpose(1, 0, 2)).reshape(total, HKV * D)
        v = np.ascontiguousarray(kv[:, :, 1, :].transpose(1, 0, 2)).reshape(total, HKV * D)
        yield prefix, suffix, q, gate, k, v


def host_cache(prefix: int, suffix: int, k: np.ndarray, v: np.ndarray, mode: int):
    """The test's cache of one mode (0 fp16/fp16, 1 q8 K, 2 q8 V, 3 q8 K and V; one scale per row, the test's quantiser)."""
    host = ko.HostCache(prefix + suffix + 128, HKV, D, D, mode)
    host.append(k, v, None, 0, rope_mode=0, quant_style=1)
    return host


def run_cases(count: int):
    out = []
    for prefix, suffix, q, gate, k, v in draw_cases(count):
        outputs = {mode: host_cache(prefix, suffix, k, v, mode).suffix_splitk(q, gate, prefix, SCALE, num_splits=32) for mode in (0, 1, 2, 3)}
        out.append({"prefix": prefix, "suffix": suffix, "q8_k": metrics(outputs[0], outputs[1]),
                    "q8_v": metrics(outputs[0], outputs[2]), "q8_kv": metrics(outputs[0], outputs[3])})
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", type=int, default=4)
    args = ap.parse_args()
    ko.set_threads(os.cpu_count() or 1)
    result = {"recipe": "tests/qwen3_quant_kv_attention_test.cpp:79-154 of the reference, through the CPU oracle",
              "published": {"source": "experiments/EXP-V2-0024-quantized-prefix-kv.md:122-126 of the reference",
                            "max_abs": 0.001263, "mae": 0.000011, "cos": 0.999973},
              "cases": run_cases(args.cases)}
    path = Path(__file__).with_name("quant_kv_attention_pin.json")
    path.write_text(json.dumps(result, indent=1) + "\n")
    print(path)
