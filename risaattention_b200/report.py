"""Benchmark report files in the layout of the reference's ``schema_version`` 2 JSON.

The reference's benchmark scripts save one JSON document per run (benchmarks/common.py:251-360):
an envelope with the environment and the run's configuration, a list of result records -- one per
(case, seed, implementation, V mode, stage) with a timing summary -- and, for every pair of records
that differ only in the V mode, the latency and error change from absmax to midpoint-affine.  Tools
written against those files (plots, regression checks) read this module's output unchanged.
"""
from __future__ import annotations

import hashlib
import importlib.metadata
import json
import statistics
from datetime import datetime, timezone
from pathlib import Path

SCHEMA_VERSION = 2
V_MODES = ("absmax", "midpoint_affine")
_PAIRING_KEYS = ("implementation", "case", "shape", "seed", "layout", "qk_distribution",
                 "value_distribution", "stage")


def _quantile(values, fraction):
    """Linear interpolation between order statistics, ``fraction`` in [0, 1]."""
    ordered = sorted(values)
    if not ordered:
        raise ValueError("no samples")
    position = fraction * (len(ordered) - 1)
    low = int(position)
    high = min(low + 1, len(ordered) - 1)
    return ordered[low] + (ordered[high] - ordered[low]) * (position - low)


def timing_summary(samples_ms, *, calls_per_sample, warmup):
    """Median, 10th and 90th percentile of per-call times (ms), with the raw samples."""
    samples_ms = [float(x) for x in samples_ms]
    return {"median_ms": statistics.median(samples_ms), "p10_ms": _quantile(samples_ms, 0.1),
            "p90_ms": _quantile(samples_ms, 0.9), "samples_ms": samples_ms,
            "calls_per_sample": int(calls_per_sample), "warmup": int(warmup)}


def result_record(*, case, shape, seed, implementation, v_quantization, stage, timing,
                  accuracy=None, memory=None, sparse=None, layout="hnd", qk_distribution="normal",
                  value_distribution="normal"):
    """One measurement.  ``shape``: dict of the case's sizes; ``stage``: what was timed (``full``
    = quantisation + attention, ``attention`` = packed operands only, ``construct``, ``sparse``)."""
    return {"case": case, "shape": dict(shape), "seed": seed, "layout": layout,
            "qk_distribution": qk_distribution, "value_distribution": value_distribution,
            "implementation": implementation, "v_quantization": v_quantization, "stage": stage,
            "timing": timing, "accuracy": accuracy, "memory": memory, "sparse": sparse}


def _percent_change(before, after):
    return None if before in (None, 0) or after is None else 100.0 * (after - before) / before


def midpoint_affine_comparisons(results):
    """For records that differ only in the V mode: change from absmax to midpoint-affine."""
    by_setting: dict = {}
    for row in results:
        if row["v_quantization"] not in V_MODES:
            continue
        setting = json.dumps([row[key] for key in _PAIRING_KEYS], sort_keys=True)
        by_setting.setdefault(setting, {})[row["v_quantization"]] = row
    out = []
    for modes in by_setting.values():
        if len(modes) != 2:
            continue
        off, on = modes["absmax"], modes["midpoint_affine"]
        entry = {key: off[key] for key in _PAIRING_KEYS}
        entry["latency_change_percent"] = _percent_change(off["timing"]["median_ms"],
                                                          on["timing"]["median_ms"])
        entry["nrmse_change_percent"] = (
            _percent_change(off["accuracy"]["nrmse"], on["accuracy"]["nrmse"])
            if off["accuracy"] and on["accuracy"] else None)
        out.append(entry)
    return out


def _file_digest(paths):
    digest = hashlib.sha256()
    for path in sorted(paths):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def environment():
    """GPU, toolkit and library identity of the measuring process."""
    import torch

    from . import __version__, _backend

    package = Path(__file__).resolve().parent
    sources = [p for p in package.rglob("*")
               if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".h") and "_obj" not in p.parts]
    versions = {}
    for name in ("torch", "sageattention", "comfy-kitchen"):
        try:
            versions[name] = importlib.metadata.version(name)
        except importlib.metadata.PackageNotFoundError:
            versions[name] = None
    cuda = torch.cuda.is_available()
    return {"gpu": torch.cuda.get_device_name() if cuda else None,
            "capability": list(torch.cuda.get_device_capability()) if cuda else None,
            "cuda": torch.version.cuda, "versions": versions, "risa_version": __version__,
            "package_path": str(package / "__init__.py"),
            "source_sha256": _file_digest(sources),
            "extension_sha256": hashlib.sha256(Path(_backend._LIB_PATH).read_bytes()).hexdigest()}


def build_report(suite, config, results, *, environment_info=None,
                 reference="FP32 PyTorch SDPA, query chunks limited to 16M score elements"):
    return {"schema_version": SCHEMA_VERSION, "suite": suite,
            "measured_at_utc": datetime.now(timezone.utc).isoformat(),
            "environment": environment() if environment_info is None else environment_info,
            "config": dict(config), "reference": reference, "results": list(results),
            "affine_comparisons": midpoint_affine_comparisons(results)}


def write_report(path, suite, config, results, **kwargs):
    """Writes the document (NaN is refused, as in the reference's writer) and returns its path."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(build_report(suite, config, results, **kwargs), indent=2,
                               allow_nan=False) + "\n")
    return path
