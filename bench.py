#!/usr/bin/env python
"""Benchmark of the quantised-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--seq-len 32768] [--scaling strong|weak] [--no-extras] [--report FILE]

Workload: the reference's dense sweep at 32K -- ``int8_attention`` on B=1, Hq=16, Hkv=4, D=128,
bf16, Lq=Lk=32768, HND contiguous, q/k/v i.i.d. N(0,1) from ``torch.Generator(seed 0)`` in the
reference's generator order (benchmarks/common.py:105-131).  A step is one full call (K anchor,
Q/K/V quantisation, fused attention).  ``value`` is dense-equivalent INT8 TOPS,
4*B*Hq*Lq*Lk*D / time (benchmarks/plot_scaling.py:66-74), with inputs resident in HBM;
``ms_per_step`` is the full-call latency.  ``e2e`` is the same metric through the public
host-operand call with the inputs in pinned host memory: the timed region copies q, k, v to the
device and the output back every step.  ``roofline`` is for the dominant kernel (the fused
attention kernel, tensor bound) timed alone with CUDA events; ``prep_roofline`` gives the HBM-bound
preparation kernels.  ``cpu_baseline`` times the CPU restatement of the path (oracle/) on a bounded
sample; ``reference_kernels_on_this_gpu`` times the reference project's own CUDA kernels
(oracle/_ref) on the same inputs when that library is present.  Further keys (N = 1 only, skipped by
``--no-extras``): ``dense_sweep`` (every length x V mode of the sweep under the reference's timing
protocol: 200 warm-up calls, 10 samples of 20 calls, median per seed, median over seeds 0/1/2),
``sparse_reuse`` on both sparse workloads, ``video_dit`` (one GPU's 5 heads at L=32760) and
``edge_sweep`` (Hq32 Hkv8 Lq4096 Lk16384, D 64 / 256).

N > 1 (launched by torchrun, one rank per GPU).  The path has no exchange step.  Default
(``--scaling strong``): ONE 32K call whose 16 query heads are split over the ranks with KV heads
co-located, or replicated when there are more ranks than KV heads (risaattention_b200/sharding.py);
``value`` = ops of the whole call / max-over-ranks time.  Extra keys: CTA waves per rank,
``gather_ms`` (NCCL all-gather of the per-rank outputs, for callers that want the result on one
device; not part of the timed step) and ``sharding_check`` (gathered output and merged sparse
pattern compared bit for bit with a single-GPU run on rank 0).  ``--scaling weak`` gives every rank
its own full 32K call instead.  Timing: max over ranks of CUDA-event time, bracketed by barriers.

``--impl reference`` times the reference's CPU path.  The reference ships no CPU implementation of
this path (its Python refuses non-CUDA tensors), so this arm runs the CPU restatement in oracle/ on
all host threads, on a bounded sample of the same workload, and reports the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

B, HQ, HKV, D = 1, 16, 4, 128
METRIC = "dense_equiv_int8_tops_32k_full_call"
# DRAM bytes (read + written) of one attention_tc_kernel launch from an ncu capture of this script,
# keyed by (sequence length, query heads on the GPU); other shapes report null.
NCU_DRAM_BYTES_PER_LAUNCH = {(32768, 16): 101901824 + 99419136}
# kernels the library launches for one unmasked dense call with absmax V: (K anchor + V range + Q),
# (K + V codes), attention
KERNELS_PER_DENSE_CALL = 3


def dense_ops(batch, heads, lq, lk, d):
    return 4.0 * batch * heads * lq * lk * d


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def make_inputs(seq_len, device, seed=0, heads=HQ, kv_heads=HKV, batch=B):
    from risaattention_b200 import synthetic

    return synthetic.dense_inputs(seq_len, device, seed=seed, q_heads=heads, kv_heads=kv_heads,
                                  head_dim=D, batch=batch)


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    # NVML reason bits (nvml.h): sw_power_cap 0x4, hw_slowdown 0x8, sw_thermal 0x20, hw_thermal 0x40
    NVML_REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                    0x40: "hw_thermal_slowdown"}

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.thread = None
        self.samples = []

    def _poll_nvml(self, pynvml, handle):
        while not self.stop:
            try:
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
                try:
                    bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except AttributeError:
                    bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(sm), float(mx), int(bits)))
            except Exception:
                break
            time.sleep(0.005)

    def __enter__(self):
        # read-only NVML polling every 5 ms (several samples inside a 100 ms timed region);
        # nvidia-smi in a loop is the fallback
        try:
            import pynvml
            import threading
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.index
            if visible:
                entry = visible.split(",")[self.index]
                index = int(entry) if entry.isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.stop = False
            self.thread = threading.Thread(target=self._poll_nvml, args=(pynvml, handle),
                                           daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            self.stop = True
            self.thread.join(timeout=2)
            if self.samples:
                reasons = set()
                for _, _, bits in self.samples:
                    reasons.update(name for bit, name in self.NVML_REASONS.items() if bits & bit)
                self.result = {"sm_mhz": statistics.median(s[0] for s in self.samples),
                               "sm_max_mhz": max(s[1] for s in self.samples),
                               "reasons": sorted(reasons), "samples": len(self.samples),
                               "source": "nvml, 5 ms period"}
            return
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx),
                           "reasons": sorted(reasons), "samples": len(sm),
                           "source": "nvidia-smi -lms 50"}


def event_time_ms(fn, steps, warmup, barrier=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return start.elapsed_time(stop) / steps


# ---------------------------------------------------------------------------------------------
# CPU legs (the only places that execute oracle/)
# ---------------------------------------------------------------------------------------------
def cpu_sample_run(seq_len, threads, heads=4, queries=1024):
    """One bounded sample of the workload on the host: `heads` query heads of one KV head,
    `queries` query rows, all keys.  Returns (seconds, ops)."""
    from oracle import risa_oracle as O

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, heads, queries, D, generator=g).bfloat16()
    k = torch.randn(1, 1, seq_len, D, generator=g).bfloat16()
    v = torch.randn(1, 1, seq_len, D, generator=g).bfloat16()
    t0 = time.perf_counter()
    O.int8_attention(q, k, v)
    return time.perf_counter() - t0, dense_ops(1, heads, queries, seq_len, D)


def cpu_baseline(seq_len):
    threads = os.cpu_count() or 1
    seconds, ops = cpu_sample_run(seq_len, threads)
    return {"value": ops / seconds / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"CPU restatement (oracle/risa_oracle.py), 4 query heads x 1024 queries x "
                      f"{seq_len} keys of one KV head incl. quantisation: {seconds:.2f} s"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_sample_run(args.seq_len, threads, heads=1, queries=128)
    times, ops = [], 0.0
    for _ in range(args.steps):
        seconds, ops = cpu_sample_run(args.seq_len, threads, heads=2, queries=512)
        times.append(seconds)
    seconds = sum(times) / len(times)
    value = ops / seconds / 1e12
    full_ms = seconds * 1e3 * dense_ops(B, HQ, args.seq_len, args.seq_len, D) / ops
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_ms,
        "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 and args.scaling == "strong" else "weak",
        "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": f"dense int8_attention B{B} Hq{HQ} Hkv{HKV} D{D} L{args.seq_len} bf16",
                   "note": "reference has no CPU path; CPU restatement timed; ms_per_step is the "
                           "sample time scaled to the full workload"},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": "port",
                         "sample": f"2 query heads x 512 queries x {args.seq_len} keys per step"},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def reference_kernels_leg(q, k, v, seq_len, steps):
    """The reference project's own CUDA kernels (compiled into oracle/_ref) on the same inputs."""
    try:
        from oracle import ref_gpu
        if not ref_gpu.available():
            return None
        cta_k = 128 if seq_len > 1024 else 64
        pk = ref_gpu.prequantize(q, k, v, cta_k=cta_k)
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)

        def full():
            p = ref_gpu.prequantize(q, k, v, cta_k=cta_k)
            ref_gpu.attention(p, sm_scale=D ** -0.5, out=out)

        ms_full = event_time_ms(full, max(2, steps // 2), 2)
        ms_att = event_time_ms(lambda: ref_gpu.attention(pk, sm_scale=D ** -0.5, out=out),
                               max(2, steps // 2), 1)
        ops = dense_ops(q.shape[0], q.shape[1], seq_len, seq_len, D)
        return {"full_call_ms": ms_full, "attention_ms": ms_att, "tops": ops / ms_full / 1e9,
                "what": "reference CUDA kernels (mma.sync path) built for sm_100, same inputs"}
    except Exception as error:  # comparison leg only
        return {"error": str(error)[:200]}


def accuracy_leg(q, k, v, out_ours, seq_len):
    """NRMSE against FP32 softmax attention on one query head per KV head (all queries, all keys),
    for this library and, when built, for the reference's kernels on the same inputs."""
    group = q.shape[1] // k.shape[1]
    heads = list(range(0, q.shape[1], group))
    want = torch.empty(q.shape[0], len(heads), seq_len, D, device=q.device)
    chunk = 2048
    for i, h in enumerate(heads):
        kf = k[:, h // group].float()
        vf = v[:, h // group].float()
        for start in range(0, seq_len, chunk):
            qf = q[:, h, start:start + chunk].float() * D ** -0.5
            want[:, i, start:start + chunk] = torch.softmax(qf @ kf.transpose(-1, -2), -1) @ vf

    def nrmse(x):
        x = x[:, heads].float()
        return float(((x - want).pow(2).mean() / want.pow(2).mean()).sqrt())

    result = {"heads_checked": heads, "nrmse_vs_fp32_sdpa": nrmse(out_ours)}
    try:
        from oracle import ref_gpu
        if ref_gpu.available():
            cta_k = 128 if seq_len > 1024 else 64
            ref_out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
            ref_gpu.attention(ref_gpu.prequantize(q, k, v, cta_k=cta_k), sm_scale=D ** -0.5,
                              out=ref_out)
            result["reference_kernels_nrmse"] = nrmse(ref_out)
            # parity rule of the tests: |ours - ref| <= 2e-3 RMS + one bf16 unit in the last place
            a, b = out_ours.float(), ref_out.float()
            ulp = torch.maximum(a.abs(), b.abs()) * 2.0 ** -7
            rms = b.pow(2).mean().sqrt()
            result["max_abs_beyond_one_bf16_ulp_over_rms"] = float(
                ((a - b).abs() - ulp).clamp_min(0).max() / rms)
            result["fraction_of_elements_differing"] = float((a != b).float().mean())
    except Exception as error:  # comparison only
        result["reference_error"] = str(error)[:200]
    return result


def sparse_leg(seq_len, device, steps, workload="video_blocks"):
    import risaattention_b200 as risa
    from risaattention_b200 import synthetic

    if workload == "video_blocks":
        q, k, v, g = synthetic.video_block_inputs(seq_len, device)
    else:
        q, k, v, g = synthetic.block_centroid_inputs(seq_len, device)
    _, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99)
    construct_ms = event_time_ms(
        lambda: risa.construct_sparse_int8_attention(q, k, v, theta=0.99), max(2, steps // 2), 2)
    kind = "additive" if workload == "video_blocks" else "blend"
    q2, k2, v2 = (synthetic.drift(t, g, kind) for t in (q, k, v))
    sparse_ms = event_time_ms(lambda: risa.sparse_int8_attention(q2, k2, v2, pattern), steps, 3)
    dense_ms = event_time_ms(lambda: risa.int8_attention(q2, k2, v2), steps, 3)
    return {"seq_len": seq_len, "theta": 0.99, "coverage": pattern.coverage,
            "construct_ms": construct_ms, "sparse_ms": sparse_ms, "dense_ms": dense_ms,
            "construct_over_dense": construct_ms / dense_ms,
            "speedup_vs_dense": dense_ms / sparse_ms,
            "inputs": ("reference generator: 2 alternating prototypes of norm 8 per KV head added to "
                       "N(0,1) Q/K, additive drift 0.05" if workload == "video_blocks" else
                       "per-128-token-block centroids + 0.5 N(0,1); reuse on 0.95 x + 0.05 N(0,1)")}


def reference_protocol_ms(fn, warmup=200, samples=10, calls=20, keep=None):
    """The reference's timing protocol (benchmarks/common.py:184-220): warm-up calls, then
    `samples` timings of `calls` back-to-back calls between CUDA events; returns the median.
    `keep`: optional list that receives the per-sample times."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(samples):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(calls):
            fn()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) / calls)
    if keep is not None:
        keep.extend(times)
    return statistics.median(times)


def dense_sweep_leg(device, lengths=(512, 1024, 2048, 4096, 8192, 16384, 32768), seeds=(0, 1, 2),
                    records=None):
    """Full-call latency of every (length, V mode) of the dense sweep, median over seeds of the
    per-seed median, next to the reference's own CUDA kernels on the same inputs (shorter
    protocol for those: 20 warm-ups, 5 samples of 10 calls)."""
    import risaattention_b200 as risa

    try:
        from oracle import ref_gpu
        have_ref = ref_gpu.available()
    except Exception:
        have_ref = False
    rows = []
    for length in lengths:
        for mode in ("absmax", "midpoint_affine"):
            ours, theirs = [], []
            for seed in seeds:
                q, k, v = make_inputs(length, device, seed=seed)
                # long sequences need fewer warm-ups to reach steady clocks than 200 x 7 ms
                warm = 200 if length <= 8192 else 50
                samples = []
                ours.append(reference_protocol_ms(
                    lambda: risa.int8_attention(q, k, v, v_quantization=mode), warmup=warm,
                    keep=samples))
                if records is not None:  # one report record per (length, seed, V mode)
                    from risaattention_b200 import report

                    records.append(report.result_record(
                        case=f"L{length}", seed=seed, implementation="risa_b200",
                        v_quantization=mode, stage="full",
                        shape={"batch": B, "q_heads": HQ, "kv_heads": HKV, "q_length": length,
                               "kv_length": length, "head_dim": D},
                        timing=report.timing_summary(samples, calls_per_sample=20, warmup=warm)))
                if have_ref and seed == seeds[0]:
                    cta_k = 128 if length > 1024 else 64
                    out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)

                    def ref_call():
                        pk = ref_gpu.prequantize(q, k, v, cta_k=cta_k,
                                                 midpoint_affine=mode == "midpoint_affine")
                        ref_gpu.attention(pk, sm_scale=D ** -0.5, out=out)

                    theirs.append(reference_protocol_ms(ref_call, warmup=20, samples=5, calls=10))
            ms = statistics.median(ours)
            row = {"seq_len": length, "v_quantization": mode, "ms": ms,
                   "tops": dense_ops(B, HQ, length, length, D) / ms / 1e9}
            if theirs:
                row["reference_kernels_ms"] = theirs[0]
            rows.append(row)
    return {"protocol": "200 warm-up calls (50 above 8K), 10 samples x 20 calls, median per seed, "
                        "median over seeds 0/1/2; reference kernels driven by ctypes, seed 0, 20 "
                        "warm-ups, 5 x 10 calls",
            "rows": rows}


def video_dit_leg(device, steps):
    """One GPU's share of the video-DiT configuration (5 of 40 heads, Hq = Hkv, L = 32760):
    dense call, pattern construction and sparse reuse at theta = 0.99."""
    import risaattention_b200 as risa
    from risaattention_b200 import synthetic

    heads, length = 5, 32760
    q, k, v = synthetic.video_dit_inputs(heads, device, seq_len=length)
    dense_ms = event_time_ms(lambda: risa.int8_attention(q, k, v), steps, 3)
    _, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99)
    construct_ms = event_time_ms(
        lambda: risa.construct_sparse_int8_attention(q, k, v, theta=0.99), max(2, steps // 2), 2)
    sparse_ms = event_time_ms(lambda: risa.sparse_int8_attention(q, k, v, pattern), steps, 3)
    result = {"heads_per_gpu": heads, "seq_len": length, "dense_ms": dense_ms,
              "dense_tops": dense_ops(1, heads, length, length, D) / dense_ms / 1e9,
              "construct_ms": construct_ms, "coverage": pattern.coverage, "sparse_ms": sparse_ms}
    try:
        from oracle import ref_gpu
        if ref_gpu.available():
            out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)

            def ref_call():
                ref_gpu.attention(ref_gpu.prequantize(q, k, v, cta_k=128), sm_scale=D ** -0.5,
                                  out=out)

            result["reference_kernels_dense_ms"] = event_time_ms(ref_call, max(2, steps // 2), 2)
    except Exception as error:  # comparison only
        result["reference_error"] = str(error)[:200]
    return result


def edge_sweep_leg(device, steps):
    """Edge / feature sweep timings at Hq32 Hkv8 Lq4096 Lk16384 for head_dim 64 and 256."""
    import risaattention_b200 as risa
    from risaattention_b200 import synthetic

    rows = []
    for dim in (64, 256):
        for feature in ("dense_b2_lse", "causal", "bias_mask", "bool_mask_rows"):
            batch = 2 if feature in ("dense_b2_lse", "bool_mask_rows") else 1
            q, k, v = synthetic.dense_inputs(4096, device, seed=dim, q_heads=32, kv_heads=8,
                                             head_dim=dim, batch=batch, kv_len=16384)
            g = torch.Generator(device=device).manual_seed(dim + 1)
            kwargs = {}
            if feature == "causal":
                kwargs["is_causal"] = True
            elif feature == "bias_mask":
                kwargs["attn_mask"] = torch.randn(batch, 32, 4096, 16384, device=device, generator=g)
            elif feature == "bool_mask_rows":
                mask = torch.ones(batch, 32, 4096, 16384, device=device, dtype=torch.bool)
                mask[:, :, torch.randperm(4096, device=device, generator=g)[:409]] = False
                kwargs["attn_mask"] = mask
            else:
                kwargs["return_lse"] = True
            ms = event_time_ms(lambda: risa.int8_attention(q, k, v, **kwargs), max(3, steps // 2), 3)
            ops = dense_ops(batch, 32, 4096, 16384, dim) * (0.5 if feature == "causal" else 1.0)
            row = {"head_dim": dim, "feature": feature, "batch": batch, "ms": ms,
                   "tops_executed": ops / ms / 1e9}
            try:
                from oracle import ref_gpu
                if ref_gpu.available():
                    cta_k = 64 if ("attn_mask" in kwargs or dim == 64) else 128
                    mask = kwargs.get("attn_mask")
                    out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)

                    def ref_call():
                        pk = ref_gpu.prequantize(q, k, v, cta_k=cta_k)
                        ref_gpu.attention(pk, sm_scale=dim ** -0.5, mask=mask, out=out,
                                          is_causal=kwargs.get("is_causal", False),
                                          want_lse=feature == "dense_b2_lse")

                    row["reference_kernels_ms"] = event_time_ms(ref_call, 3, 2)
            except Exception as error:  # comparison only
                row["reference_error"] = str(error)[:120]
            rows.append(row)
            del kwargs
    return rows


def mma_issue_loop_tops(device):
    """INT8 tensor-pipe ceiling of this GPU at its current clocks, from the probe library (built
    beside the product library; see include/risa_b200_probe.h): back-to-back kind::i8 128x256x32
    MMAs on every SM, no loads."""
    import ctypes

    path = ROOT / "risaattention_b200" / "librisa_b200_probe.so"
    if not path.exists():
        return None
    lib = ctypes.CDLL(str(path))
    fn = lib.risa_b200_mma_i8_issue_loop
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    ctas, ops = ctypes.c_int(0), ctypes.c_double(0.0)
    stream = torch.cuda.current_stream(device).cuda_stream

    def launch():
        if fn(8192, ctypes.byref(ctas), ctypes.byref(ops), stream) != 0:
            raise RuntimeError("INT8 issue-loop probe failed to launch")

    ms = event_time_ms(launch, 10, 3)
    return ops.value / ms / 1e9


def tail_split_parts(ctas, key_tiles, sms, cta_k=128):
    """Key-range parts per CTA of the last wave in the one-call dense path (0: whole CTAs), asked
    of the library itself."""
    from risaattention_b200 import _backend

    return int(_backend._ABI.lib.risa_b200_split_last_wave_parts(ctas, key_tiles, cta_k, sms))


def cta_waves(q_heads_local, seq_len, sms=None):
    if sms is None:
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    ctas = q_heads_local * ((seq_len + 127) // 128)
    parts = tail_split_parts(ctas, (seq_len + 127) // 128, sms)
    rest = ctas % sms
    # the last wave: whole CTAs, or ceil(rest * parts / sms) rounds of 1 / parts of a CTA's time
    waves = ctas // sms + (-(-rest * parts // sms) / parts if parts else float(rest > 0))
    return {"ctas": ctas, "sms": sms, "waves": ctas / sms,
            "last_wave_key_range_parts": parts,
            "wave_efficiency": (ctas / sms) / waves}


def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: dist.barrier(device_ids=[local_rank])  # noqa: E731

    import risaattention_b200 as risa
    from risaattention_b200 import _backend
    from risaattention_b200.sharding import gather_heads, merge_patterns, plan_head_shard

    L = args.seq_len
    sharded = args.scaling == "strong" and world > 1
    shard = None
    if sharded:
        shard = plan_head_shard(HQ, HKV, rank, world)
        full_q, full_k, full_v = make_inputs(L, device, seed=0)
        q = full_q[:, shard.q_start:shard.q_stop].contiguous()
        k = full_k[:, shard.kv_start:shard.kv_stop].contiguous()
        v = full_v[:, shard.kv_start:shard.kv_stop].contiguous()
        if rank != 0:
            del full_q, full_k, full_v
        total_ops = dense_ops(B, HQ, L, L, D)
        parallelism = (f"one call, {HQ // world} query heads per GPU, KV heads co-located"
                       f"{' (replicated across GPU pairs)' if world > HKV else ''}, no collective")
    else:
        q, k, v = make_inputs(L, device, seed=rank)
        total_ops = dense_ops(B, HQ, L, L, D) * world
        parallelism = f"{world} independent calls, one {L}-token call per GPU, no collective" \
            if world > 1 else "single GPU"
    local_ops = dense_ops(q.shape[0], q.shape[1], L, L, D)

    def step():
        return risa.int8_attention(q, k, v)

    with ClockSampler(local_rank) as clocks:
        ms = event_time_ms(step, args.steps, args.warmup, barrier)
    _backend._C.device_status()
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)

    # ---- end to end: pinned host inputs, output read back, every step -------------------------
    # (each rank moves only the heads it owns)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    host_out = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        # public host-operand entry point: one stage per KV head, PCIe copies overlapped with
        # compute; the timed region ends with a device synchronisation, so the output is complete
        risa.int8_attention_from_host(hq, hk, hv, out=host_out, device=device, wait=False)

    e2e_ms = event_time_ms(e2e_step, max(2, args.steps // 2), 3, barrier)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = host_out.numel() * host_out.element_size()
    if world > 1:
        moved = torch.tensor([h2d, d2h], device=device, dtype=torch.int64)
        dist.all_reduce(moved)
        h2d, d2h = int(moved[0]), int(moved[1])

    extra = {}
    if sharded:
        # output reassembly for callers that want one device to hold the result: NCCL all-gather
        local_out = step()
        gather_ms = event_time_ms(lambda: gather_heads(local_out), 5, 2, barrier)
        t = torch.tensor([gather_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gathered = gather_heads(local_out)
        # sparse supports: construct on the shard, merge in global row order
        ls, kl = min(L, 8192), None
        sq = q[:, :, :ls].contiguous()
        sk, sv = k[:, :, :ls].contiguous(), v[:, :, :ls].contiguous()
        _, local_pattern = risa.construct_sparse_int8_attention(sq, sk, sv, theta=0.9)
        merged_offsets, merged_indices = merge_patterns(local_pattern.row_offsets,
                                                        local_pattern.block_indices, B)
        check = None
        if rank == 0:
            want = risa.int8_attention(full_q, full_k, full_v)
            _, full_pattern = risa.construct_sparse_int8_attention(
                full_q[:, :, :ls].contiguous(), full_k[:, :, :ls].contiguous(),
                full_v[:, :, :ls].contiguous(), theta=0.9)
            # rows of a split last wave (parts of the key range merged afterwards) may differ from
            # the unsplit single-GPU rows in the last place; everything else is the same bits
            differ = (gathered != want)
            rms = want.float().pow(2).mean().sqrt()
            check = {"gathered_output_bit_identical_to_single_gpu": bool(torch.equal(gathered, want)),
                     "gathered_output_fraction_differing": float(differ.float().mean()),
                     "gathered_output_max_abs_over_rms":
                         float((gathered.float() - want.float()).abs().max() / rms),
                     "merged_pattern_bit_identical_to_single_gpu":
                         bool(torch.equal(merged_offsets, full_pattern.row_offsets)
                              and torch.equal(merged_indices, full_pattern.block_indices)),
                     "pattern_seq_len": ls}
        extra = {"gather_ms": float(t),
                 "gather_bytes_per_rank": local_out.numel() * local_out.element_size(),
                 "cta_waves_per_rank": cta_waves(q.shape[1], L),
                 "sharding_check": check}

    if rank != 0:
        if world > 1:
            dist.barrier(device_ids=[local_rank])
            dist.destroy_process_group()
        return

    # ---- kernel-level roofline legs (rank 0) -------------------------------------------------------
    peaks = measured_peaks()
    packed = risa.prequantize_int8_attention(q, k, v)
    att_ms = event_time_ms(lambda: risa.int8_attention_from_prequantized(packed), args.steps,
                           args.warmup)
    prep_ms = event_time_ms(lambda: risa.prequantize_int8_attention(q, k, v), args.steps,
                            args.warmup)
    int8_peak = 2.0 * peaks["bf16_tflops"]  # no INT8 entry in MEASURED_PEAKS: 2 x measured bf16
    mma_loop_tops = mma_issue_loop_tops(device)
    achieved = local_ops / att_ms / 1e9
    prep_bytes = sum(t.numel() * 3 for t in (q, k, v))  # 2 B in + 1 B out per element
    line = {
        "metric": METRIC, "value": total_ops / ms / 1e9, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
        "config": {"workload": f"dense int8_attention B{B} Hq{HQ} Hkv{HKV} D{D} L{L} bf16, "
                               "full call incl. Q/K/V quantisation",
                   "parallelism": parallelism,
                   "l2": "inputs + packed operands (>300 MB at 32K) exceed the 126 MB L2"},
        "clocks": clocks.result,
        "e2e": {"value": total_ops / e2e_ms / 1e9, "unit": "TOPS", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        # the merge launch of a split last wave counts when the shape takes it
        "gpu_launches": (KERNELS_PER_DENSE_CALL
                         + (cta_waves(q.shape[1], L)["last_wave_key_range_parts"] > 0))
                        * args.steps * world,
        "roofline": {"bound": "tensor", "kernel": "attention_tc_kernel", "achieved": achieved,
                     "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
                     "kernel_ms": att_ms,
                     "peak_source": f"2 x {peaks['source']} bf16 {peaks['bf16_tflops']} TFLOP/s "
                                    "(no INT8 figure in MEASURED_PEAKS.json)",
                     "peak_int8_issue_loop": mma_loop_tops,
                     "frac_of_issue_loop": None if not mma_loop_tops else achieved / mma_loop_tops,
                     "peak_int8_issue_loop_source": "measured in this run by this repository's own "
                                                    "probe kernel: back-to-back tcgen05.mma kind::i8 "
                                                    "128x256x32 on every SM, no loads",
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((L, q.shape[1])),
                     "traffic_source": "constant: dram__bytes_read.sum + dram__bytes_write.sum of one "
                                       "launch of this workload from an ncu capture, not measured in "
                                       "this run"},
        "prep_roofline": {"bound": "hbm", "achieved": prep_bytes / prep_ms / 1e6,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": prep_bytes / prep_ms / 1e6 / peaks["hbm_gbs"],
                          "kernel_ms": prep_ms,
                          "note": f"{KERNELS_PER_DENSE_CALL - 1} kernels incl. host launch gaps"},
    }
    line.update(extra)
    if world == 1:
        line["accuracy"] = accuracy_leg(q, k, v, step(), L)
        line["reference_kernels_on_this_gpu"] = reference_kernels_leg(q, k, v, L, args.steps)
        line["cta_waves"] = cta_waves(q.shape[1], L)
        del packed
        if not args.no_extras:
            half = max(3, args.steps // 2)
            records = [] if args.report else None
            for key, leg in (("sparse_reuse", lambda: sparse_leg(L, device, half)),
                             ("sparse_reuse_block_centroids",
                              lambda: sparse_leg(L, device, half, "block_centroids")),
                             ("dense_sweep", lambda: dense_sweep_leg(device, records=records)),
                             ("video_dit", lambda: video_dit_leg(device, half)),
                             ("edge_sweep", lambda: edge_sweep_leg(device, half))):
                try:
                    line[key] = leg()
                except Exception as error:  # an extra must never cost the headline line
                    line[key] = {"error": str(error)[:200]}
                torch.cuda.empty_cache()
            if args.report and records:
                from risaattention_b200 import report

                config = {"layout": "hnd", "samples": 10, "calls_per_sample": 20,
                          "timing_order": "one implementation per pass", "seeds": [0, 1, 2],
                          "dtype": "bfloat16"}
                report.write_report(args.report, "dense_sweep", config, records)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(L)
    print(json.dumps(line))
    if world > 1:
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="N > 1: split one call's heads over the ranks (strong, default) or run "
                         "one full call per rank (weak)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--report", default=None,
                    help="also write the dense sweep as a schema_version 2 report (the reference's "
                         "benchmark file layout) to this path")
    ap.add_argument("--no-extras", "--no-sparse", dest="no_extras", action="store_true",
                    help="skip the sparse-reuse, dense-sweep, video-DiT and edge-sweep legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
