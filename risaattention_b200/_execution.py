"""Dense and prequantised attention execution: validation of packed operands, sparse patterns and
capture workspaces, output allocation and the native call
(reference src/risa_attention/_execution.py:28-328)."""
from __future__ import annotations

import math

import torch

from . import _backend
from ._key_mask import prepare_key_mask_tiles
from ._quantization import (PackedBuffers, pad_head_dim, quantize_into, resolve_scale)
from ._types import PrequantizedInt8Attention, RetainedMassPattern
from ._validation import (DTYPE_CODES, MIN_PATTERN_SPARSITY, OUTPUT_LAYOUTS, UNAVAILABLE,
                          is_available, mask_signature, select_key_block_size, validate_inputs)


def _output_dtype(input_dtype):
    return torch.bfloat16 if input_dtype == torch.float32 else input_dtype


def execute_dense_attention(q, k, v, *, scale=None, attn_mask=None, use_midpoint_affine=False,
                            is_causal=False):
    """Single-call path: quantise and attend on the current stream; scratch lives only for the call."""
    attn_mask = validate_inputs(q, k, v, attn_mask)
    input_dtype = q.dtype
    q, k, v, original_head_dim, dim = pad_head_dim(q, k, v)
    attention_scale = resolve_scale(scale, original_head_dim)
    batch, q_heads, q_len, _ = q.shape
    key_block_size = select_key_block_size(
        dim, k.shape[2], has_mask=attn_mask is not None and attn_mask.stride(-2) != 0)
    out_dtype = _output_dtype(input_dtype)
    output = torch.empty(batch, q_heads, q_len, dim, dtype=out_dtype, device=q.device)
    stream = _backend.current_stream_ptr(q.device)
    if attn_mask is None:
        # one native call, one scratch allocation: what bounds short sequences is the host side
        scratch = torch.empty(
            _backend._C.dense_scratch_size(batch, q_heads, q_len, k.shape[1], k.shape[2], dim,
                                           key_block_size), dtype=torch.uint8, device=q.device)
        _backend._C.risa_dense_attention(q, k, v, output, scratch, key_block_size,
                                         DTYPE_CODES[input_dtype], use_midpoint_affine,
                                         attention_scale, DTYPE_CODES[out_dtype], is_causal, stream)
    else:
        buffers = PackedBuffers(q, k, key_block_size)
        tiles = prepare_key_mask_tiles(attn_mask, key_block_size, q_len, attention_scale,
                                       is_causal)
        quantize_into(buffers, q, k, v, key_block_size, use_midpoint_affine)
        _backend._C.risa_sdpa_prequantized(
            buffers.q_codes, buffers.k_codes, buffers.v_codes, output, buffers.q_scales,
            buffers.k_scales, buffers.v_scales, buffers.v_centers, key_block_size,
            attention_scale, DTYPE_CODES[out_dtype], stream, attn_mask=attn_mask,
            is_causal=is_causal, key_mask_tiles=tiles)
    if original_head_dim != dim:
        output = output[..., :original_head_dim]
    return output.float() if input_dtype == torch.float32 else output


def _check_pattern(quantized, pattern):
    if not isinstance(pattern, RetainedMassPattern):
        raise TypeError("sparse_pattern must be returned by build_retained_mass_pattern")
    if pattern.is_causal != quantized.is_causal:
        raise ValueError("sparse pattern and attention call must use the same is_causal")
    if pattern.mask_signature != mask_signature(quantized.attn_mask):
        raise ValueError("sparse pattern mask has changed; rebuild the pattern")
    expected = (quantized.q.shape[0], quantized.q.shape[1], quantized.q.shape[2],
                quantized.k.shape[2], 128, quantized.cta_k)
    actual = (pattern.batch_size, pattern.q_heads, pattern.q_length, pattern.kv_length,
              pattern.query_block_size, pattern.key_block_size)
    if actual != expected:
        raise ValueError("sparse pattern metadata does not match packed attention: "
                         f"expected {expected}, got {actual}")
    if not math.isclose(pattern.attention_scale, quantized.attention_scale, rel_tol=1e-7,
                        abs_tol=0.0):
        raise ValueError("sparse pattern and attention call must use the same scale")
    device = quantized.q.device
    if pattern.row_offsets.device != device or pattern.block_indices.device != device:
        raise ValueError("sparse pattern and packed tensors must be on the same CUDA device")
    for index in (pattern.row_offsets, pattern.block_indices):
        if index.dtype != torch.int32 or not index.is_contiguous():
            raise TypeError("sparse CSR row offsets and block indices must be contiguous int32")


def allocate_output(quantized, output_layout):
    """Output tensor of a packed call: logical [batch, heads, seq, head_dim], stored heads-major
    ("hnd") or sequence-major ("nhd")."""
    batch, q_heads, q_len, dim = quantized.q.shape
    out_dtype = _output_dtype(quantized.input_dtype)
    device = quantized.q.device
    if output_layout == "nhd":
        return torch.empty(batch, q_len, q_heads, dim, dtype=out_dtype,
                           device=device).permute(0, 2, 1, 3)
    return torch.empty(batch, q_heads, q_len, dim, dtype=out_dtype, device=device)


def finish_output(output, quantized):
    """Drops head-dim padding and restores FP32 for FP32 callers."""
    if quantized.original_head_dim != output.shape[-1]:
        output = output[..., :quantized.original_head_dim]
    return output.float() if quantized.input_dtype == torch.float32 else output


def capture_workspace_elements(quantized) -> int:
    batch, q_heads, q_len, _ = quantized.q.shape
    tiles = math.ceil(quantized.k.shape[2] / quantized.cta_k)
    return batch * q_heads * (math.ceil(q_len / 128) * tiles + q_len * (tiles * 2 + 2))


def int8_attention_from_prequantized(quantized, *, sparse_pattern=None, output_layout="hnd",
                                     _block_mass=None, return_lse=False):
    """Attend over packed operands.  Both layouts return a logical [batch, heads, seq, head_dim]
    tensor; ``"nhd"`` stores sequence before heads so ``out.transpose(1, 2).reshape(b, n, -1)`` is a
    view when the head dimension needed no padding."""
    if not isinstance(quantized, PrequantizedInt8Attention):
        raise TypeError("quantized must be returned by prequantize_int8_attention, got "
                        f"{type(quantized).__name__}")
    if output_layout not in OUTPUT_LAYOUTS:
        raise ValueError(f"output_layout must be one of {OUTPUT_LAYOUTS}, got {output_layout!r}")
    if quantized.kv_permuted and (sparse_pattern is not None or _block_mass is not None):
        raise ValueError("permuted K/V is supported only by dense attention")
    if return_lse and quantized.lse_shift is None:
        raise ValueError("prequantize with return_lse=True to retain the K-anchor correction")
    device = quantized.q.device
    packed = (quantized.k, quantized.v, quantized.q_scale, quantized.k_scale, quantized.v_scale,
              quantized.v_center)
    if not quantized.q.is_cuda:
        raise ValueError("prequantized INT8 attention tensors must be on a CUDA device")
    if any(t.device != device for t in packed):
        raise ValueError("prequantized INT8 attention tensors must be on the same CUDA device")
    if quantized.attn_mask is not None and quantized.attn_mask.device != device:
        raise ValueError("attn_mask must be on the same CUDA device as the packed tensors")
    if sparse_pattern is not None:
        _check_pattern(quantized, sparse_pattern)
        if sparse_pattern.sparsity < MIN_PATTERN_SPARSITY:
            sparse_pattern = None  # nearly dense support: the dense kernel is faster
    if _block_mass is not None:
        if sparse_pattern is not None:
            raise ValueError("block mass requires dense attention")
        expected = capture_workspace_elements(quantized)
        if (_block_mass.ndim != 1 or _block_mass.numel() != expected
                or _block_mass.dtype != torch.float32 or _block_mass.device != device
                or not _block_mass.is_contiguous()):
            raise ValueError(
                f"block mass workspace must be contiguous CUDA float32 with {expected} elements")
    if not is_available(device):
        raise RuntimeError(UNAVAILABLE)

    batch, q_heads, q_len, dim = quantized.q.shape
    out_dtype = _output_dtype(quantized.input_dtype)
    output = allocate_output(quantized, output_layout)
    lse = torch.empty((batch, q_heads, q_len), dtype=torch.float32, device=device) \
        if return_lse else None
    tiles = None
    if sparse_pattern is None and _block_mass is None:
        tiles = prepare_key_mask_tiles(quantized.attn_mask, quantized.cta_k, q_len,
                                       quantized.attention_scale, quantized.is_causal)
    _backend._C.risa_sdpa_prequantized(
        quantized.q, quantized.k, quantized.v, output, quantized.q_scale, quantized.k_scale,
        quantized.v_scale, quantized.v_center, quantized.cta_k, quantized.attention_scale,
        DTYPE_CODES[out_dtype], _backend.current_stream_ptr(device),
        attn_mask=quantized.attn_mask,
        sparse_row_offsets=None if sparse_pattern is None else sparse_pattern.row_offsets,
        sparse_block_indices=None if sparse_pattern is None else sparse_pattern.block_indices,
        block_mass=_block_mass, is_causal=quantized.is_causal, lse=lse, key_mask_tiles=tiles)
    output = finish_output(output, quantized)
    if return_lse:
        lse.add_(quantized.lse_shift)
        return output, lse
    return output
