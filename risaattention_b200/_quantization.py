"""Q/K/V preparation: padding, packed-buffer allocation and the native quantisation call
(reference src/risa_attention/_quantization.py:23-198)."""
from __future__ import annotations

import math

import torch
from torch.nn import functional

from . import _backend
from ._types import PrequantizedInt8Attention
from ._validation import (DTYPE_CODES, kernel_head_dim, pad_key_length, select_key_block_size,
                          uses_centered_values, validate_inputs)


class PackedBuffers:
    """Device buffers of one call in the public packed layouts (all caller-side allocations; the
    native library never allocates)."""

    def __init__(self, q, k, key_block_size):
        batch, q_heads, q_len, dim = q.shape
        kv_heads, k_len = k.shape[1], k.shape[2]
        dev = q.device
        self.padded_key_length = pad_key_length(k_len, key_block_size)
        allocate = getattr(_backend._C, "allocate_packed", None)
        if allocate is not None:
            # the C++ module hands out all nine buffers in one call: a third less host time for
            # a short call than nine allocations from here
            (self.q_codes, self.k_codes, self.q_scales, self.k_scales, self.v_codes,
             self.v_scales, self.v_centers, self.anchors, self.workspace) = allocate(
                 q, k, key_block_size)
            return
        self.q_codes = torch.empty(q.shape, dtype=torch.int8, device=dev)
        self.k_codes = torch.empty(k.shape, dtype=torch.int8, device=dev)
        self.q_scales = torch.empty(batch, q_heads, -(-q_len // 128) * (64 if dim == 256 else 32),
                                    dtype=torch.float32, device=dev)
        self.k_scales = torch.empty(batch, kv_heads, -(-k_len // key_block_size) * 4,
                                    dtype=torch.float32, device=dev)
        self.v_codes = torch.empty(batch * kv_heads * dim, self.padded_key_length,
                                   dtype=torch.int8, device=dev)
        self.v_scales = torch.empty(batch * kv_heads * dim, dtype=torch.float32, device=dev)
        self.v_centers = torch.empty_like(self.v_scales)
        self.anchors = torch.empty(batch, kv_heads, dtype=torch.int32, device=dev)
        self.workspace = torch.empty(
            _backend._C.quantize_v_workspace_size(batch, kv_heads, k_len, dim), dtype=torch.uint8,
            device=dev)


def pad_head_dim(q, k, v):
    original = q.shape[-1]
    target = kernel_head_dim(original)
    if target != original:
        q, k, v = (functional.pad(t, (0, target - original)) for t in (q, k, v))
    return q, k, v, original, target


def resolve_scale(scale, original_head_dim):
    value = original_head_dim ** -0.5 if scale is None else float(scale)
    if not math.isfinite(value):
        raise ValueError(f"scale must be finite, got {value}")
    return value


def quantize_into(buffers, q, k, v, key_block_size, use_midpoint_affine, kv_table=None):
    """``kv_table``: optional int32 [B,Hkv,Lk] gather table the K and V quantisers read through."""
    _backend._C.risa_sdpa_quantize(
        q, k, v, buffers.q_codes, buffers.q_scales, buffers.k_codes, buffers.k_scales,
        buffers.v_codes, buffers.v_scales, buffers.v_centers, key_block_size,
        DTYPE_CODES[q.dtype], use_midpoint_affine,
        _backend.current_stream_ptr(q.device), buffers.anchors, kv_table,
        workspace=buffers.workspace)


def prequantize_int8_attention(q, k, v, *, scale=None, attn_mask=None, v_quantization="absmax",
                               is_causal=False, return_lse=False, kv_permutation=None,
                               fuse_gather=True) -> PrequantizedInt8Attention:
    """Quantise Q, K and V on the current stream without allocating the attention output.

    The result keeps no floating-point input, so callers may free Q/K/V before
    :func:`int8_attention_from_prequantized`.  No host synchronisation is introduced."""
    attn_mask = validate_inputs(q, k, v, attn_mask)
    kv_table = None
    if kv_permutation is not None:
        from .permutation import prepare_inputs

        q, k, v, kv_table = prepare_inputs(q, k, v, permutation=kv_permutation, mask=attn_mask,
                                           causal=is_causal, return_lse=return_lse,
                                           fuse=fuse_gather)
    use_midpoint_affine = uses_centered_values(v_quantization)
    input_dtype = q.dtype
    q, k, v, original_head_dim, _ = pad_head_dim(q, k, v)
    attention_scale = resolve_scale(scale, original_head_dim)
    key_block_size = select_key_block_size(
        q.shape[-1], k.shape[2], has_mask=attn_mask is not None and attn_mask.stride(-2) != 0)
    buffers = PackedBuffers(q, k, key_block_size)
    quantize_into(buffers, q, k, v, key_block_size, use_midpoint_affine, kv_table)
    lse_shift = None
    if return_lse:
        # K was translated by its anchor row before quantisation; this restores the row-wise logit
        # offset so LSE values of different key windows can be merged.
        lse_shift = torch.empty(q.shape[:3], device=q.device, dtype=torch.float32)
        _backend._C.risa_lse_shift(q, k, buffers.anchors, lse_shift, attention_scale,
                                   _backend.current_stream_ptr(q.device))
    return PrequantizedInt8Attention(
        q=buffers.q_codes, k=buffers.k_codes, v=buffers.v_codes, q_scale=buffers.q_scales,
        k_scale=buffers.k_scales, v_scale=buffers.v_scales, v_center=buffers.v_centers,
        original_head_dim=original_head_dim, input_dtype=input_dtype,
        attention_scale=attention_scale, cta_k=key_block_size, attn_mask=attn_mask,
        v_quantization=v_quantization, is_causal=is_causal, lse_shift=lse_shift,
        kv_permuted=kv_permutation is not None)
