"""The benchmark report writer: the reference's schema_version 2 layout (benchmarks/common.py:
251-360) from this package's measurements."""
import json

import pytest

from risaattention_b200 import report


def _record(mode, samples, seed=0, nrmse=None):
    return report.result_record(
        case="L1024", seed=seed, implementation="risa_b200", v_quantization=mode, stage="full",
        shape={"batch": 1, "q_heads": 16, "kv_heads": 4, "q_length": 1024, "kv_length": 1024,
               "head_dim": 128},
        timing=report.timing_summary(samples, calls_per_sample=20, warmup=200),
        accuracy=None if nrmse is None else {"nrmse": nrmse})


def test_timing_summary_percentiles():
    t = report.timing_summary([5.0, 1.0, 3.0, 2.0, 4.0], calls_per_sample=20, warmup=200)
    assert t["median_ms"] == 3.0
    assert t["p10_ms"] == pytest.approx(1.4)
    assert t["p90_ms"] == pytest.approx(4.6)
    assert t["samples_ms"] == [5.0, 1.0, 3.0, 2.0, 4.0]
    assert (t["calls_per_sample"], t["warmup"]) == (20, 200)


def test_report_layout_and_pairing(tmp_path):
    results = [_record("absmax", [2.0, 2.0, 2.0], nrmse=0.016),
               _record("midpoint_affine", [2.1, 2.1, 2.1], nrmse=0.015),
               _record("absmax", [2.0], seed=1)]  # no partner: not compared
    env = {"gpu": "test", "capability": [10, 0]}
    path = report.write_report(tmp_path / "out" / "dense.json", "dense_sweep",
                               {"layout": "hnd"}, results, environment_info=env)
    doc = json.loads(path.read_text())
    assert doc["schema_version"] == 2 and doc["suite"] == "dense_sweep"
    assert set(doc) == {"schema_version", "suite", "measured_at_utc", "environment", "config",
                        "reference", "results", "affine_comparisons"}
    assert len(doc["results"]) == 3
    assert set(doc["results"][0]) == {"case", "shape", "seed", "layout", "qk_distribution",
                                      "value_distribution", "implementation", "v_quantization",
                                      "stage", "timing", "accuracy", "memory", "sparse"}
    (pair,) = doc["affine_comparisons"]
    assert pair["seed"] == 0 and pair["case"] == "L1024"
    assert pair["latency_change_percent"] == pytest.approx(5.0)
    assert pair["nrmse_change_percent"] == pytest.approx(-6.25)


def test_nan_is_refused(tmp_path):
    bad = [_record("absmax", [float("nan")])]
    with pytest.raises(ValueError):
        report.write_report(tmp_path / "bad.json", "dense_sweep", {}, bad, environment_info={})
