"""The two-library comparison tool end to end: a byte copy of the library under another path is a
separate image in the process, gives the same bits, and the run is written as a report."""
import json
import shutil

import pytest

pytestmark = pytest.mark.gpu

from risaattention_b200 import _backend, compare_native  # noqa: E402


def test_a_copy_of_the_library_compares_equal_and_is_timed(tmp_path):
    copy = tmp_path / "librisa_b200.so"
    shutil.copy(_backend._LIB_PATH, copy)
    out = tmp_path / "comparison.json"
    results = compare_native.main([
        "--baseline-library", str(copy), "--case", "1,4,2,300,1300,128", "--case",
        "2,2,2,128,200,64", "--seed", "0", "--samples", "2", "--calls", "2", "--warmup", "1",
        "--include-components", "--report", str(out)])
    # 2 cases x 2 V modes x 3 stages x 2 libraries
    assert len(results) == 24
    document = json.loads(out.read_text())
    assert document["schema_version"] == 2 and document["suite"] == "native-comparison"
    assert document["config"]["baseline_library_sha256"] == document["environment"]["extension_sha256"]
    assert {r["implementation"] for r in document["results"]} == {"before", "after"}
    assert {r["stage"] for r in document["results"]} == {"dense", "quantize", "prequantized_dense"}
    for record in document["results"]:
        assert record["timing"]["median_ms"] > 0 and len(record["timing"]["samples_ms"]) == 2
        assert (record["accuracy"] is None) == (record["stage"] == "quantize")
    assert len(document["affine_comparisons"]) == 12
    _backend._C.device_status()


def test_differing_bits_stop_the_run(tmp_path):
    """A library whose results differ is reported before anything is timed: here the `baseline`
    forces the row-per-thread kernel, whose outputs agree with the tensor-core kernel's only
    within tolerance."""
    import torch

    class OtherKernel:
        def __init__(self, native):
            self._native = native

        def __getattr__(self, name):
            entry = getattr(self._native, name)
            if name not in ("risa_sdpa_prequantized", "risa_dense_attention"):
                return entry

            def forced(*args, **kwargs):
                previous = self._native.set_attention_path(1)
                try:
                    return entry(*args, **kwargs)
                finally:
                    self._native.set_attention_path(previous)
            return forced

    shape = compare_native.parse_case("1,4,2,300,1300,128")
    with pytest.raises(RuntimeError, match="output bits differ"), torch.inference_mode():
        compare_native.compare(OtherKernel(_backend._ABI), _backend._ABI, [shape], [0],
                               samples=2, calls=1, warmup=0, log=lambda *a: None)
