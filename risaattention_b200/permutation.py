"""Token permutations of K and V (reference src/risa_attention/permutation.py:8-52).

A caller that clusters or re-orders its keys hands over one gather table per (batch, KV head):
row ``i`` of the attention's K/V is row ``table[i]`` of the tensors passed in.  Softmax attention is
invariant under a joint permutation of K and V, so the table only matters for how the packed
operands are laid out (K scale groups, V storage groups, the sampled anchor rows).  The quantisers
read K and V *through* the table (``fuse_gather=True``), so no gathered copy of K and V is ever
written; here that holds for every input dtype and head dim (the reference fuses bf16 / D=128 only).
"""
from __future__ import annotations

import torch

_INT32_MAX = 2**31 - 1


class KVPermutation:
    """An int32 ``[B, Hkv, Nkv]`` gather table that has been checked to be a permutation per row.

    The check sorts the table and reads the verdict back (one host synchronisation), so build the
    object once, outside any CUDA-graph capture, and reuse it.  The object owns a private copy of
    the indices and remembers the copy's version counter: an in-place write to it afterwards is
    detected at use and rejected."""

    __slots__ = ("_indices", "_version")

    def __init__(self, indices: torch.Tensor):
        if indices.ndim != 3 or indices.dtype not in (torch.int32, torch.int64):
            raise ValueError("permutation must be [B,Hkv,Nkv] int32/int64")
        if not indices.is_cuda or indices.numel() == 0:
            raise ValueError("permutation must be a nonempty CUDA tensor")
        tokens = indices.shape[-1]
        if tokens > _INT32_MAX:
            raise ValueError("permutation is too long for INT32")
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("prepare the permutation before CUDA graph capture")
        # a row is a permutation of 0..n-1 exactly when its sorted values are 0..n-1
        ramp = torch.arange(tokens, device=indices.device, dtype=indices.dtype)
        if not bool((indices.sort(dim=-1).values == ramp).all()):
            raise ValueError("each permutation row must contain each token exactly once")
        with torch.inference_mode(False):  # a normal tensor, so that its version counter works
            private = indices.to(dtype=torch.int32, copy=True).contiguous()
        object.__setattr__(self, "_indices", private)
        object.__setattr__(self, "_version", private._version)

    def __setattr__(self, name, value):
        raise AttributeError("KVPermutation is immutable")

    def table(self) -> torch.Tensor:
        """The validated int32 table; raises if it was written to after validation."""
        if self._indices._version != self._version:
            raise ValueError("validated permutation was modified")
        return self._indices


def prepare_kv_permutation(indices: torch.Tensor) -> KVPermutation:
    """Validates (synchronises once) and copies a caller-supplied permutation."""
    return KVPermutation(indices)


def prepare_inputs(q, k, v, *, permutation, mask, causal, return_lse, fuse):
    """Resolves a permutation for the quantisers: returns ``(q, k, v, table)`` where ``table`` is
    the gather table the K and V quantisers should read through, or ``None`` after K and V have
    been gathered into new tensors (``fuse=False``, or LSE output, whose anchor correction reads
    the gathered K itself)."""
    if not isinstance(permutation, KVPermutation):
        raise TypeError("use prepare_kv_permutation to validate a permutation first")
    table = permutation.table()
    if table.device != k.device or tuple(table.shape) != tuple(k.shape[:3]):
        raise ValueError("permutation must match K batch, heads, length, and device")
    if mask is not None or causal:
        raise ValueError("K/V permutation requires dense, unmasked, noncausal attention")
    if fuse and not return_lse:
        return q, k, v, table
    rows = table.to(torch.int64).unsqueeze(-1).expand(k.shape)
    return q, torch.gather(k, 2, rows), torch.gather(v, 2, rows), None
