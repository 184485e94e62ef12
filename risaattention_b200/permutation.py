"""Validated K/V token permutations (reference src/risa_attention/permutation.py:8-52): the
quantisers can read K and V through a gather table instead of materialised gathered copies."""
from dataclasses import dataclass

import torch


@dataclass(frozen=True, init=False)
class KVPermutation:
    """Owned int32 [B, Hkv, Nkv] permutation, validated once (synchronises) before graph capture."""

    _indices: torch.Tensor
    _version: int

    def __init__(self, indices: torch.Tensor):
        if indices.ndim != 3 or indices.dtype not in (torch.int32, torch.int64):
            raise ValueError("permutation must be [B,Hkv,Nkv] int32/int64")
        if not indices.is_cuda or indices.numel() == 0:
            raise ValueError("permutation must be a nonempty CUDA tensor")
        if indices.shape[-1] > 2**31 - 1:
            raise ValueError("permutation is too long for INT32")
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("prepare the permutation before CUDA graph capture")
        identity = torch.arange(indices.shape[-1], device=indices.device)
        if not torch.equal(indices.sort(-1).values, identity.expand_as(indices)):
            raise ValueError("each permutation row must contain each token exactly once")
        with torch.inference_mode(False):
            owned = indices.to(torch.int32).clone().contiguous()
        object.__setattr__(self, "_indices", owned)
        object.__setattr__(self, "_version", owned._version)


def prepare_kv_permutation(indices: torch.Tensor) -> KVPermutation:
    return KVPermutation(indices)


def prepare_inputs(q, k, v, *, permutation, mask, causal, return_lse, fuse):
    """Returns q, k, v and the (q, k, v) gather tables for the quantisers.  The fused route covers
    every dtype and head dim here; LSE needs the gathered K itself, so it materialises."""
    if not isinstance(permutation, KVPermutation):
        raise TypeError("use prepare_kv_permutation to validate a permutation first")
    table = permutation._indices
    if table._version != permutation._version:
        raise ValueError("validated permutation was modified")
    if table.device != k.device or table.shape != k.shape[:3]:
        raise ValueError("permutation must match K batch, heads, length, and device")
    if mask is not None or causal:
        raise ValueError("K/V permutation requires dense, unmasked, noncausal attention")
    if fuse and not return_lse:
        return q, k, v, (None, table, table)
    index = table.long()[..., None].expand_as(k)
    return q, k.gather(2, index), v.gather(2, index), (None, None, None)
