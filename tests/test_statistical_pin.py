"""Pins the quantized path of the oracle against figures the reference published.

The reference has no stored vectors and no CPU code for int8 K/V attention; what it has is a GPU test with a fixed
recipe (tests/qwen3_quant_kv_attention_test.cpp:79-154: std::mt19937(42), normal(0, 0.5), a host quantiser, four
(prefix, suffix) cases, errors of the quantised cache modes against the fp16 one) and an experiment record that quotes
what that test measured (experiments/EXP-V2-0024-quantized-prefix-kv.md:122-126: max-abs 0.001263, MAE 0.000011,
cosine 0.999973).  Here the oracle runs the recipe on the same random stream: the first three cases live, the fourth
(minutes of CPU) from the committed fixture that tests/golden/make_statistical_pin.py writes with the same code."""
import importlib.util
import json
import os
from pathlib import Path

import kvoracle as ko

GOLDEN = Path(__file__).parent / "golden"


def _generator():
    spec = importlib.util.spec_from_file_location("make_statistical_pin", GOLDEN / "make_statistical_pin.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_quantized_attention_errors_reproduce_the_published_figures():
    fixture = json.loads((GOLDEN / "quant_kv_attention_pin.json").read_text())
    ko.set_threads(min(os.cpu_count() or 1, 32))
    live = _generator().run_cases(3)
    cases = fixture["cases"]
    assert [(c["prefix"], c["suffix"]) for c in cases] == [(64, 16), (512, 64), (4096, 128), (16384, 512)]
    # the committed fixture is what this code computes (cases 1-3 recomputed here)
    for got, want in zip(live, cases):
        for mode in ("q8_k", "q8_v", "q8_kv"):
            for key in ("max_abs", "mae", "rmse", "cos"):
                assert abs(got[mode][key] - want[mode][key]) <= 1e-9 * max(1.0, abs(want[mode][key])), (want["prefix"], mode, key)
    # the reference's own acceptance gate for the path, every case and mode (.cpp:271)
    for c in cases:
        assert min(c[m]["cos"] for m in ("q8_k", "q8_v", "q8_kv")) >= 0.999 and c["q8_kv"]["mae"] <= 0.05
    # the published figures, to the digits the record prints: the largest error over the cases (it is the first
    # case's), the cosine of that case, and the mean error of the longest case
    pub = fixture["published"]
    assert (pub["max_abs"], pub["mae"], pub["cos"]) == (0.001263, 0.000011, 0.999973)
    both = [c["q8_kv"] for c in cases]
    assert round(max(m["max_abs"] for m in both), 6) == pub["max_abs"]
    assert round(both[0]["cos"], 6) == pub["cos"]
    assert round(both[3]["mae"], 6) == pub["mae"]
    # and the errors fall with the context length, as averaging over more positions makes them
    assert both[0]["mae"] > both[1]["mae"] > both[2]["mae"] > both[3]["mae"]
