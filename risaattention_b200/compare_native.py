"""Compare a preserved build of the kernel library with the current one on identical inputs.

For changes that are meant to keep every output bit.  Both libraries are loaded into one process;
every case is first checked for equality (the outputs, and with ``--include-components`` each
packed operand), only then both are timed, with their positions in the measurement order balanced
so that neither always runs first, and the run is saved in the benchmark report layout
(:mod:`risaattention_b200.report`).  The reference keeps the same tool for two builds of its
extension module (benchmarks/compare_native.py:34-152).  Here the preserved build is a copy of
``librisa_b200.so`` kept under another path: the C++ extension module is linked against the
library by name, so a second copy of the *module* would resolve to the library that is already
loaded; a second copy of the *library* opened by path through the ctypes surface
(:class:`risaattention_b200._backend._Native`) is a separate image.  To compare like with like the
current library is driven through the same ctypes surface.

    python -m risaattention_b200.compare_native --baseline-library /keep/librisa_b200.so \\
        --case 1,16,4,4096,4096,128 --include-components --report comparison.json
"""
from __future__ import annotations

import argparse
import hashlib
from pathlib import Path

import torch

from . import _backend, report

V_MODES = ("absmax", "midpoint_affine")
PACKED_FIELDS = ("q", "k", "v", "q_scale", "k_scale", "v_scale", "v_center")


def parse_case(text: str) -> dict:
    """``"B,Hq,Hkv,Lq,Lk,D"`` -> the sizes of one case."""
    parts = text.split(",")
    if len(parts) != 6:
        raise argparse.ArgumentTypeError("a case is B,Hq,Hkv,Lq,Lk,D")
    try:
        batch, q_heads, kv_heads, q_len, k_len, head_dim = (int(p) for p in parts)
    except ValueError as error:
        raise argparse.ArgumentTypeError("a case is six integers: B,Hq,Hkv,Lq,Lk,D") from error
    if min(batch, q_heads, kv_heads, q_len, k_len, head_dim) <= 0 or q_heads % kv_heads:
        raise argparse.ArgumentTypeError("sizes must be positive and Hq a multiple of Hkv")
    return {"batch": batch, "q_heads": q_heads, "kv_heads": kv_heads, "q_len": q_len,
            "k_len": k_len, "head_dim": head_dim}


def case_label(shape: dict) -> str:
    return "B{batch}_Hq{q_heads}_Hkv{kv_heads}_Lq{q_len}_Lk{k_len}_D{head_dim}".format(**shape)


def load_library(path):
    """The ctypes surface over the library file at ``path`` (a separate image when the file is not
    the one already loaded)."""
    path = Path(path).resolve()
    if not path.is_file():
        raise FileNotFoundError(f"no library at {path}")
    return _backend._Native(path)


def with_native(native, function):
    """Runs ``function()`` with every call of the package routed to ``native``."""
    original = _backend._C
    _backend._C = native
    try:
        return function()
    finally:
        _backend._C = original


def balanced_orders(names, samples: int):
    """Measurement order of each sample: forwards and backwards in turn, so that over an even
    number of samples every method has run in every position equally often with its mirror."""
    names = list(names)
    return [names if sample % 2 == 0 else names[::-1] for sample in range(samples)]


def measure_methods(methods: dict, *, samples: int, calls: int, warmup: int) -> dict:
    """Per-call times of every method from CUDA events around ``calls`` back-to-back calls,
    ``samples`` times in balanced order after ``warmup`` untimed calls of each."""
    for function in methods.values():
        for _ in range(warmup):
            function()
    torch.cuda.synchronize()
    times = {name: [] for name in methods}
    for order in balanced_orders(methods, samples):
        for name in order:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(calls):
                methods[name]()
            stop.record()
            stop.synchronize()
            times[name].append(start.elapsed_time(stop) / calls)
    return {name: report.timing_summary(values, calls_per_sample=calls, warmup=warmup)
            for name, values in times.items()}


def make_inputs(shape: dict, seed: int, dtype=torch.bfloat16, device="cuda"):
    """q, k, v ~ N(0,1) from one generator in that order (the dense benchmark's inputs)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def normal(heads, length):
        return torch.randn(shape["batch"], heads, length, shape["head_dim"], device=device,
                           generator=g).to(dtype)

    return (normal(shape["q_heads"], shape["q_len"]), normal(shape["kv_heads"], shape["k_len"]),
            normal(shape["kv_heads"], shape["k_len"]))


def _accuracy(output, q, k, v):
    """NRMSE against FP32 attention, computed per query head to bound the score matrix."""
    group = q.shape[1] // k.shape[1]
    error = torch.zeros((), dtype=torch.float64, device=q.device)
    power = torch.zeros((), dtype=torch.float64, device=q.device)
    for head in range(q.shape[1]):
        want = torch.nn.functional.scaled_dot_product_attention(
            q[:, head:head + 1].float(), k[:, head // group:head // group + 1].float(),
            v[:, head // group:head // group + 1].float())
        error += (output[:, head:head + 1].float() - want).double().pow(2).sum()
        power += want.double().pow(2).sum()
    return {"nrmse": float((error / power.clamp_min(1e-30)).sqrt())}


def compare(baseline, current, cases, seeds, modes=V_MODES, *, include_components=False,
            samples=24, calls=20, warmup=20, log=print):
    """Equality first, timing second.  Returns the result records; raises ``RuntimeError`` at the
    first tensor whose bits differ between the two libraries."""
    import risaattention_b200 as risa

    results = []
    for shape in cases:
        label = case_label(shape)
        for seed in seeds:
            q, k, v = make_inputs(shape, seed)
            methods, errors, tags = {}, {}, {}
            for mode in modes:

                def dense(mode=mode):
                    return risa.int8_attention(q, k, v, v_quantization=mode)

                before, after = with_native(baseline, dense), with_native(current, dense)
                if not torch.equal(before, after):
                    raise RuntimeError(f"output bits differ: {label}, seed {seed}, {mode}")
                error = _accuracy(after, q, k, v)
                stages = {"dense": dense}
                if include_components:

                    def quantize(mode=mode):
                        return risa.prequantize_int8_attention(q, k, v, v_quantization=mode)

                    packs = [with_native(native, quantize) for native in (baseline, current)]
                    for field in PACKED_FIELDS:
                        if not torch.equal(getattr(packs[0], field), getattr(packs[1], field)):
                            raise RuntimeError(
                                f"packed {field} bits differ: {label}, seed {seed}, {mode}")
                    outputs = [with_native(native, lambda pack=pack:
                                           risa.int8_attention_from_prequantized(pack))
                               for native, pack in zip((baseline, current), packs)]
                    if not torch.equal(outputs[0], outputs[1]):
                        raise RuntimeError(
                            f"prequantized output bits differ: {label}, seed {seed}, {mode}")
                    stages["quantize"] = quantize
                    stages["prequantized_dense"] = (
                        lambda pack=packs[0]: risa.int8_attention_from_prequantized(pack))
                for stage, operation in stages.items():
                    for side, native in (("before", baseline), ("after", current)):
                        name = f"{side}/{mode}/{stage}"
                        methods[name] = (lambda native=native, operation=operation:
                                         with_native(native, operation))
                        errors[name] = None if stage == "quantize" else error
                        tags[name] = (side, mode, stage)
            timings = measure_methods(methods, samples=samples, calls=calls, warmup=warmup)
            for name, (side, mode, stage) in tags.items():
                results.append(report.result_record(
                    case=label, shape=shape, seed=seed, implementation=side, v_quantization=mode,
                    stage=stage, timing=timings[name], accuracy=errors[name]))
            log(label, seed, {name: round(t["median_ms"], 6) for name, t in timings.items()})
    return results


def build_parser():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--baseline-library", required=True, type=Path,
                        help="preserved copy of librisa_b200.so")
    parser.add_argument("--case", action="append", type=parse_case, help="B,Hq,Hkv,Lq,Lk,D")
    parser.add_argument("--seed", action="append", type=int)
    parser.add_argument("--v-quantization", action="append", choices=V_MODES)
    parser.add_argument("--include-components", action="store_true",
                        help="also compare and time quantisation and attention on packed operands")
    parser.add_argument("--samples", type=int, default=24)
    parser.add_argument("--calls", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--report", type=Path, help="write the run as a schema_version 2 report")
    return parser


@torch.inference_mode()
def main(argv=None):
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.samples < 2 or args.samples % 2 or args.calls < 1 or args.warmup < 0:
        parser.error("--samples must be even and at least 2, --calls positive, --warmup >= 0")
    if _backend._ABI is None:
        raise RuntimeError(f"the current library did not load: {_backend._EXTENSION_ERROR}")
    cases = args.case or [parse_case("1,16,4,512,512,128")]
    seeds = args.seed or [0, 1, 2]
    modes = tuple(args.v_quantization or V_MODES)
    baseline = load_library(args.baseline_library)
    current = _backend._ABI
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    results = compare(baseline, current, cases, seeds, modes,
                      include_components=args.include_components, samples=args.samples,
                      calls=args.calls, warmup=args.warmup)
    if args.report:
        config = {"cases": [case_label(c) for c in cases], "seeds": seeds,
                  "v_quantization": list(modes), "include_components": args.include_components,
                  "samples": args.samples, "calls": args.calls, "warmup": args.warmup,
                  "baseline_library": str(args.baseline_library.resolve()),
                  "baseline_library_sha256": hashlib.sha256(
                      args.baseline_library.read_bytes()).hexdigest()}
        report.write_report(args.report, "native-comparison", config, results)
    return results


if __name__ == "__main__":
    main()
