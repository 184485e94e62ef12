#!/usr/bin/env python
"""Benchmark of the quantised-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--seq-len 32768] [--scaling weak|strong]

Workload (N = 1): the reference's dense sweep at 32K -- ``int8_attention`` on B=1, Hq=16, Hkv=4,
D=128, bf16, Lq=Lk=32768, HND contiguous, q/k/v i.i.d. N(0,1) from ``torch.Generator(seed 0)`` in
the reference's generator order (benchmarks/common.py:105-131).  A step is one full call (K anchor,
Q/K/V quantisation, fused attention).  ``value`` is dense-equivalent INT8 TOPS,
4*B*Hq*Lq*Lk*D / time (benchmarks/plot_scaling.py:66-74), with inputs resident in HBM;
``ms_per_step`` is the full-call latency.  ``e2e`` is the same metric through the public API with
the inputs in pinned host memory: the timed region copies q, k, v to the device and the output back
every step.  ``roofline`` is for the dominant kernel (the fused attention kernel, tensor bound)
timed alone with CUDA events; ``prep_roofline`` gives the HBM-bound preparation kernels.
``cpu_baseline`` times the CPU restatement of the path (oracle/) on a bounded sample;
``reference_kernels_on_this_gpu`` times the reference project's own CUDA kernels (oracle/_ref)
on the same inputs when that library is present.  Extra keys report sparse reuse.

N > 1 (launched by torchrun, one rank per GPU): the path has no exchange step.  ``--scaling weak``
(default) gives every rank its own 32K call (global batch N); ``--scaling strong`` splits the 16
query heads of one call over the ranks with KV heads co-located (risaattention_b200/sharding.py).
Timing: max over ranks of CUDA-event time, bracketed by barriers.

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
NCU_DRAM_BYTES_PER_LAUNCH = {(32768, 16): 101529856 + 81629696}


def dense_ops(batch, heads, lq, lk, d):
    return 4.0 * batch * heads * lq * lk * d


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def make_inputs(seq_len, device, seed=0, heads=HQ, kv_heads=HKV, batch=B):
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(batch, heads, seq_len, D, device=device, generator=g).bfloat16()
    k = torch.randn(batch, kv_heads, seq_len, D, device=device, generator=g).bfloat16()
    v = torch.randn(batch, kv_heads, seq_len, D, device=device, generator=g).bfloat16()
    return q, k, v


def block_structured_inputs(seq_len, device, seed=0):
    """Sparse-reuse generator of the benchmark spec: one centroid per 128-token block and head,
    tokens = centroid + 0.5 N(0,1); V ~ N(0,1)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def blocks(heads):
        cent = torch.randn(B, heads, seq_len // 128, 1, D, device=device, generator=g)
        noise = torch.randn(B, heads, seq_len // 128, 128, D, device=device, generator=g)
        return (cent + 0.5 * noise).reshape(B, heads, seq_len, D).bfloat16()

    q, k = blocks(HQ), blocks(HKV)
    v = torch.randn(B, HKV, seq_len, D, device=device, generator=g).bfloat16()
    return q, k, v, g


def video_blocks_inputs(seq_len, device, seed=0, clusters=2, prototype_norm=8.0):
    """The reference's own sparse-benchmark generator (benchmarks/sparse.py:33-52): N(0,1) q/k/v
    plus, per KV head, `clusters` unit-direction prototypes of norm 8 added to Q and K by
    128-token block (block index modulo clusters)."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(B, HQ, seq_len, D, device=device, generator=g).bfloat16()
    k = torch.randn(B, HKV, seq_len, D, device=device, generator=g).bfloat16()
    v = torch.randn(B, HKV, seq_len, D, device=device, generator=g).bfloat16()
    proto = torch.randn(B, HKV, clusters, D, device=device, generator=g)
    proto *= prototype_norm / proto.norm(dim=-1, keepdim=True)
    cluster = torch.arange(seq_len, device=device).div(128, rounding_mode="floor") % clusters
    q = q + proto.repeat_interleave(HQ // HKV, dim=1)[:, :, cluster].to(q.dtype)
    k = k + proto[:, :, cluster].to(k.dtype)
    return q, k, v, g


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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
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


def sparse_leg(seq_len, device, steps, generator="video_blocks"):
    import risaattention_b200 as risa

    if generator == "video_blocks":
        q, k, v, g = video_blocks_inputs(seq_len, device)
    else:
        q, k, v, g = block_structured_inputs(seq_len, device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99)
    torch.cuda.synchronize()
    construct_ms = (time.perf_counter() - t0) * 1e3
    construct_ms = min(construct_ms, event_time_ms(
        lambda: risa.construct_sparse_int8_attention(q, k, v, theta=0.99), 2, 1))

    def drift(x):
        noise = torch.randn(x.shape, device=device, generator=g)
        if generator == "video_blocks":  # additive drift, as the reference benchmark
            return (x.float() + 0.05 * noise).bfloat16()
        return (0.95 * x.float() + 0.05 * noise).bfloat16()

    q2, k2, v2 = drift(q), drift(k), drift(v)
    sparse_ms = event_time_ms(lambda: risa.sparse_int8_attention(q2, k2, v2, pattern), steps, 3)
    dense_ms = event_time_ms(lambda: risa.int8_attention(q2, k2, v2), steps, 3)
    return {"seq_len": seq_len, "theta": 0.99, "coverage": pattern.coverage,
            "construct_ms": construct_ms, "sparse_ms": sparse_ms, "dense_ms": dense_ms,
            "speedup_vs_dense": dense_ms / sparse_ms,
            "inputs": ("reference generator: 2 alternating prototypes of norm 8 per KV head added to "
                       "N(0,1) Q/K, additive drift 0.05" if generator == "video_blocks" else
                       "per-128-token-block centroids + 0.5 N(0,1); reuse on 0.95 x + 0.05 N(0,1)")}


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
    from risaattention_b200.sharding import plan_head_shard

    L = args.seq_len
    if args.scaling == "strong" and world > 1:
        shard = plan_head_shard(HQ, HKV, rank, world)
        q, k, v = make_inputs(L, device, seed=0)
        q = q[:, shard.q_start:shard.q_stop].contiguous()
        k = k[:, shard.kv_start:shard.kv_stop].contiguous()
        v = v[:, shard.kv_start:shard.kv_stop].contiguous()
        total_ops = dense_ops(B, HQ, L, L, D)
        parallelism = f"heads sharded {HQ // world} q-heads/GPU, KV co-located, no collective"
    else:
        q, k, v = make_inputs(L, device, seed=rank)
        total_ops = dense_ops(B, HQ, L, L, D) * world
        parallelism = f"dp{world}: one {L}-token call per GPU, no collective"
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
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    host_out = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        # public host-operand entry point: one stage per KV head, PCIe copies overlapped with compute
        risa.int8_attention_from_host(hq, hk, hv, out=host_out, device=device)

    e2e_ms = event_time_ms(e2e_step, max(2, args.steps // 2), 2, barrier)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = host_out.numel() * host_out.element_size()

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
    # measured INT8 issue-loop throughput of this GPU (kind::i8 128x256x32 back to back, all SMs)
    stream_ptr = torch.cuda.current_stream(device).cuda_stream
    _, loop_ops = _backend._C.mma_i8_issue_loop(8192, stream_ptr)
    loop_ms = event_time_ms(lambda: _backend._C.mma_i8_issue_loop(8192, stream_ptr), 10, 3)
    mma_loop_tops = loop_ops / loop_ms / 1e9
    achieved = local_ops / att_ms / 1e9
    prep_bytes = sum(t.numel() * 3 for t in (q, k, v))  # 2 B in + 1 B out per element
    line = {
        "metric": METRIC, "value": total_ops / ms / 1e9, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling if world > 1 else "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
        "config": {"workload": f"dense int8_attention B{B} Hq{HQ} Hkv{HKV} D{D} L{L} bf16, "
                               "full call incl. Q/K/V quantisation",
                   "parallelism": parallelism,
                   "l2": "inputs + packed operands (>300 MB at 32K) exceed the 126 MB L2"},
        "clocks": clocks.result,
        "e2e": {"value": total_ops / e2e_ms / 1e9, "unit": "TOPS", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": 6 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "attention_tc_kernel", "achieved": achieved,
                     "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
                     "kernel_ms": att_ms,
                     "mma_i8_issue_loop_tops": mma_loop_tops,
                     "frac_of_issue_loop": achieved / mma_loop_tops,
                     "peak_source": f"2 x {peaks['source']} bf16 {peaks['bf16_tflops']} TFLOP/s "
                                    "(no INT8 figure in MEASURED_PEAKS.json)",
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((L, q.shape[1])),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, "
                                       "profiles/attention_tc_kernel_dense32k_dram_traffic.md"},
        "prep_roofline": {"bound": "hbm", "achieved": prep_bytes / prep_ms / 1e6,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": prep_bytes / prep_ms / 1e6 / peaks["hbm_gbs"],
                          "kernel_ms": prep_ms, "note": "5 kernels incl. host launch gaps"},
    }
    if world == 1:
        line["accuracy"] = accuracy_leg(q, k, v, step(), L)
        line["reference_kernels_on_this_gpu"] = reference_kernels_leg(q, k, v, L, args.steps)
        if not args.no_sparse:
            try:
                line["sparse_reuse"] = sparse_leg(L, device, max(3, args.steps // 2))
                line["sparse_reuse_block_centroids"] = sparse_leg(L, device, max(3, args.steps // 2),
                                                                  "block_centroids")
            except Exception as error:
                line["sparse_reuse"] = {"error": str(error)[:200]}
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
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sparse", action="store_true", help="skip the sparse-reuse leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
