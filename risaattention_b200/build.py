"""Builds librisa_b200.so (the C-ABI library, nvcc for sm_100a) and the PyTorch C++ extension
``_C`` over it, both in-tree.

Usage: ``python -m risaattention_b200.build [--force]``.  Objects are cached under
``risaattention_b200/csrc/_obj`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "_obj"
LIB = PKG / "librisa_b200.so"
UNITS = ["prep_qk", "prep_v", "misc", "attention_api", "attention_rows", "attention_tc"]
# measurement probe (INT8 issue-loop ceiling used by bench.py), its own library
PROBE_LIB = PKG / "librisa_b200_probe.so"
PROBE_UNITS = ["mma_peak"]
# --use_fast_math is part of the numeric contract shared with the reference's kernels
# (approximate division / reciprocal, flush-to-zero, contracted multiply-adds).
NVCC_FLAGS = [
    "-std=c++17", "-O3", "--use_fast_math", "--expt-relaxed-constexpr",
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
]


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))
    return max(p.stat().st_mtime for p in headers)


def _compile(unit: str, force: bool, verbose: bool) -> str | None:
    src, obj = CSRC / f"{unit}.cu", OBJ / f"{unit}.o"
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest_header()):
        return None
    cmd = ["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {unit}.cu:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build_torch_extension(force: bool = False) -> Path:
    """Compiles csrc/torch_binding.cpp into the in-tree module ``risaattention_b200/_C*.so``: the
    PyTorch C++ extension through which the Python runtime reaches the C-ABI library (linked by
    relative run path, so the pair can be moved together)."""
    import sysconfig

    import pybind11
    import torch
    from torch.utils import cpp_extension

    target = PKG / f"_C{sysconfig.get_config_var('EXT_SUFFIX')}"
    src = CSRC / "torch_binding.cpp"
    newest = max(src.stat().st_mtime, (PKG.parent / "include" / "risa_b200.h").stat().st_mtime)
    if not force and target.exists() and target.stat().st_mtime > newest:
        return target
    includes = [*cpp_extension.include_paths(), pybind11.get_include(),
                sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    torch_lib = str(Path(torch.__file__).resolve().parent / "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           *[f"-I{path}" for path in includes], str(src), "-o", str(target),
           f"-L{PKG}", "-lrisa_b200", f"-L{torch_lib}", "-ltorch_python", "-ltorch", "-ltorch_cpu",
           "-lc10", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"g++ failed for torch_binding.cpp:\n{proc.stdout}\n{proc.stderr}")
    return target


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    units = UNITS + PROBE_UNITS
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        logs = dict(zip(units, pool.map(lambda u: _compile(u, force, verbose), units)))
    if verbose:
        for unit, log in logs.items():
            if log:
                (OBJ / f"{unit}.ptxas.log").write_text(log)
    for lib, members in ((LIB, UNITS), (PROBE_LIB, PROBE_UNITS)):
        if any(logs[u] is not None for u in members) or not lib.exists():
            objs = [str(OBJ / f"{u}.o") for u in members]
            subprocess.run(["nvcc", "-shared", "-o", str(lib), *objs, "-lcudart"], check=True)
    build_torch_extension(force)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
