"""Attention over host-resident operands, pipelined by head group.

A caller whose Q/K/V live in (pinned) host memory pays two PCIe transfers around the kernels.  The
path is independent per (batch, KV head) -- the same property the multi-GPU sharding uses -- so the
call is cut into stages of one KV head and some of its query heads, and the stages are pipelined over
three streams: host-to-device copies of stage g+1 and the device-to-host copy of stage g-1 run while
stage g computes.  Results are identical to a single device-resident call (every stage runs the
same kernels on the same per-head data).  The reference has no counterpart: its API takes CUDA
tensors only.
"""
from __future__ import annotations

import threading

import torch

from .dense import int8_attention

_STREAMS: dict = {}
_STREAMS_LOCK = threading.Lock()


def int8_attention_from_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                             out: torch.Tensor | None = None, *, device=None,
                             wait: bool = True, heads_per_stage: int | None = None, **kwargs):
    """``int8_attention`` for CPU tensors in ``[B, H, L, D]`` layout; returns a pinned CPU tensor.

    ``kwargs`` are passed to :func:`int8_attention` (``scale``, ``is_causal``, ``v_quantization``).
    Masks, LSE and KV permutations are not supported here.  Pinned inputs make the copies
    asynchronous; pageable inputs work but serialise.

    ``heads_per_stage``: query heads per pipeline stage (default: half the query heads of a KV head);
    smaller stages overlap the copies more finely and quantise their K/V head once per stage.

    With ``wait=True`` (default) the call returns once the last device-to-host copy has finished,
    so the returned tensor can be read on the host at once.  With ``wait=False`` it returns
    ``(out, event)`` while copies may still be in flight: the host must ``event.synchronize()``
    before it reads ``out`` (work queued afterwards on the caller's stream is ordered already).
    """
    for name in ("attn_mask", "return_lse", "kv_permutation"):
        option = kwargs.get(name)
        if option is not None and option is not False:
            raise ValueError(f"int8_attention_from_host does not support {name}")
    if query.device.type != "cpu" or key.device.type != "cpu" or value.device.type != "cpu":
        raise ValueError("int8_attention_from_host expects CPU tensors")
    if query.ndim != 4 or key.shape != value.shape or query.shape[0] != key.shape[0]:
        raise ValueError("expected q [B, Hq, Lq, D] and k, v [B, Hkv, Lk, D]")
    batch, q_heads = query.shape[:2]
    kv_heads = key.shape[1]
    if q_heads % kv_heads:
        raise ValueError(f"q head count ({q_heads}) must be divisible by k/v head count ({kv_heads})")
    group = q_heads // kv_heads
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out_dtype = query.dtype
    if out is None:
        out = torch.empty(query.shape, dtype=out_dtype, pin_memory=True)
    elif out.shape != query.shape or out.device.type != "cpu" or not out.is_contiguous():
        raise ValueError("out must be a contiguous CPU tensor of q's shape")

    caller = torch.cuda.current_stream(device)
    # Two compute streams taken in turn: the last, partly filled wave of CTAs of one stage then
    # overlaps the first wave of the next stage instead of leaving SMs idle at every stage boundary.
    # The four side streams are created once per device and reused: the caching allocator keeps its
    # free blocks per stream, so fresh streams on every call would send every stage to cudaMalloc.
    with _STREAMS_LOCK:
        streams = _STREAMS.get(device)
        if streams is None:
            streams = _STREAMS[device] = tuple(torch.cuda.Stream(device) for _ in range(4))
    computes, copy_in, copy_out = streams[:2], streams[2], streams[3]
    start = torch.cuda.Event()
    start.record(caller)
    for stream in (*computes, copy_in, copy_out):
        stream.wait_event(start)  # work queued earlier on the caller's stream comes first
    # Stages: per (batch, KV head), half of its query heads each (on the 32K call with 4 query heads
    # per KV head: stages of 2 heads 8.09 ms, of 4 heads 8.25 ms, of 1 head 8.55 ms), except that the
    # very first and the very last stage of the call carry a single query head, because the upload
    # of the first stage and the download of the last one are the only transfers nothing can hide
    # (a K/V head is quantised once per stage, which costs far less than the overlap saves).
    per_stage = ((group + 1) // 2 if heads_per_stage is None
                 else max(1, min(group, int(heads_per_stage))))
    stages = []
    for b in range(batch):
        for h in range(kv_heads):
            for lo in range(h * group, (h + 1) * group, per_stage):
                stages.append((b, h, lo, min(lo + per_stage, (h + 1) * group)))
    b, h, lo, hi = stages[0]
    if hi - lo > 1:
        stages[0:1] = [(b, h, lo, lo + 1), (b, h, lo + 1, hi)]
    b, h, lo, hi = stages[-1]
    if hi - lo > 1:
        stages[-1:] = [(b, h, lo, hi - 1), (b, h, hi - 1, hi)]
    keep = []
    resident = (None, None, None)  # (batch, KV head) whose K and V are on the device, and the tensors
    for index, (b, h, lo, hi) in enumerate(stages):
        qs = slice(lo, hi)
        compute = computes[index % 2]
        with torch.cuda.stream(copy_in):
            dq = query[b:b + 1, qs].to(device, non_blocking=True)
            if resident[0] != (b, h):  # K / V travel once per KV head, also when its stage is split
                resident = ((b, h), key[b:b + 1, h:h + 1].to(device, non_blocking=True),
                            value[b:b + 1, h:h + 1].to(device, non_blocking=True))
            dk, dv = resident[1], resident[2]
            ready = torch.cuda.Event()
            ready.record(copy_in)
        compute.wait_event(ready)
        for t in (dq, dk, dv):
            t.record_stream(compute)
        with torch.cuda.stream(compute):
            result = int8_attention(dq, dk, dv, **kwargs)
            done = torch.cuda.Event()
            done.record(compute)
        copy_out.wait_event(done)
        result.record_stream(copy_out)
        with torch.cuda.stream(copy_out):
            out[b:b + 1, qs].copy_(result, non_blocking=True)
        keep.append((dq, dk, dv, result))
    finished = torch.cuda.Event()
    finished.record(copy_out)
    caller.wait_event(finished)  # the caller's stream sees the output once this event has passed
    if not wait:
        return out, finished
    finished.synchronize()
    return out
