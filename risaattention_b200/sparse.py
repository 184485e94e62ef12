"""Retained-mass pattern construction during a dense pass and sparse reuse over the frozen tile
lists (reference src/risa_attention/sparse.py:18-178)."""
from __future__ import annotations

import math

import torch

from . import _backend
from ._execution import (OUTPUT_LAYOUTS, allocate_output, capture_workspace_elements,
                         finish_output, int8_attention_from_prequantized)
from ._quantization import prequantize_int8_attention
from ._types import PrequantizedInt8Attention, RetainedMassPattern
from ._validation import DTYPE_CODES, UNAVAILABLE, is_available, mask_signature


def select_retained_mass_csr(masses: torch.Tensor, theta: float):
    """Shortest descending prefix of each row reaching ``theta`` of the row's mass, packed as CSR
    with ascending tile ids.  Returns (row_offsets, block_indices, measured retained mass); reads
    the three-number summary back, which synchronises the stream."""
    rows, tiles = masses.shape
    dev = masses.device
    sorted_mass, order = masses.sort(dim=-1, descending=True)
    counts = torch.empty(rows, dtype=torch.int32, device=dev)
    support = torch.empty((rows, tiles), dtype=torch.uint8, device=dev)
    row_totals = torch.empty(rows, 2, dtype=torch.float64, device=dev)
    row_offsets = torch.empty(rows + 1, dtype=torch.int32, device=dev)
    storage = torch.empty(rows * tiles, dtype=torch.int32, device=dev)
    summary = torch.empty(3, dtype=torch.float64, device=dev)
    scratch = torch.empty(_backend._C.retained_mass_selector_workspace_size(rows),
                          dtype=torch.uint8, device=dev)
    _backend._C.select_retained_mass_csr(sorted_mass, order, counts, support, row_totals,
                                         row_offsets, storage, summary, scratch, theta,
                                         _backend.current_stream_ptr(dev))
    selected_mass, total_mass, selected_blocks = summary.tolist()
    return row_offsets, storage[: int(selected_blocks)], selected_mass / max(total_mass, 1e-20)


def _selects_in_pass(quantized, k_blocks) -> bool:
    """True when the attention kernel itself can reduce the block masses and close the retained
    prefix: tensor-core kernel shapes with a bounded number of key tiles."""
    if quantized.kv_permuted or not quantized.q.is_cuda:
        return False
    padded = quantized.v.shape[1]
    return padded >= 128 and k_blocks <= _backend._C.select_max_key_tiles(quantized.cta_k)


def _construct_in_pass(quantized, theta, output_layout, rows, k_blocks):
    """One attention launch that also emits, per query block, the kept-tile bitmap and count, then
    one small launch that packs them as CSR.  The only host synchronisation is the read of the
    three-number summary (kept mass, total mass, kept tiles)."""
    device = quantized.q.device
    if not is_available(device):
        raise RuntimeError(UNAVAILABLE)
    native = _backend._C
    stream = _backend.current_stream_ptr(device)
    output = allocate_output(quantized, output_layout)
    counts = torch.empty(rows, dtype=torch.int32, device=device)
    bitmaps = torch.empty(rows, (k_blocks + 31) // 32, dtype=torch.int32, device=device)
    totals = torch.empty(rows, 2, dtype=torch.float64, device=device)
    scratch = torch.empty(native.select_scratch_size(quantized.k.shape[2], quantized.cta_k),
                          dtype=torch.uint8, device=device)
    native.risa_sdpa_select(
        quantized.q, quantized.k, quantized.v, output, quantized.q_scale, quantized.k_scale,
        quantized.v_scale, quantized.v_center, quantized.cta_k, quantized.attention_scale,
        DTYPE_CODES[output.dtype], stream, float(theta), scratch, counts, bitmaps, totals,
        attn_mask=quantized.attn_mask, is_causal=quantized.is_causal)
    row_offsets = torch.empty(rows + 1, dtype=torch.int32, device=device)
    storage = torch.empty(rows * k_blocks, dtype=torch.int32, device=device)
    summary = torch.empty(3, dtype=torch.float64, device=device)
    native.pack_selected(counts, bitmaps, totals, row_offsets, storage, summary, k_blocks, stream)
    selected_mass, total_mass, selected_blocks = summary.tolist()
    return (finish_output(output, quantized), row_offsets, storage[: int(selected_blocks)],
            selected_mass / max(total_mass, 1e-20))


@torch.inference_mode()
def construct_sparse_int8_attention_from_prequantized(quantized, *, theta=0.99,
                                                      output_layout="hnd"):
    """Dense attention over packed operands that also records, per 128-query block, the probability
    mass of every key tile (from the kernel's own U8 probabilities) and keeps the tiles that hold
    ``theta`` of it."""
    if not 0.0 < theta <= 1.0 or not math.isfinite(theta):
        raise ValueError("theta must be finite and in (0, 1]")
    if not isinstance(quantized, PrequantizedInt8Attention):
        raise TypeError("quantized must be returned by prequantize_int8_attention, got "
                        f"{type(quantized).__name__}")
    if output_layout not in OUTPUT_LAYOUTS:
        raise ValueError(f"output_layout must be one of {OUTPUT_LAYOUTS}, got {output_layout!r}")
    batch, q_heads, q_len, _ = quantized.q.shape
    q_blocks = math.ceil(q_len / 128)
    k_blocks = math.ceil(quantized.k.shape[2] / quantized.cta_k)
    if _selects_in_pass(quantized, k_blocks):
        output, row_offsets, block_indices, measured = _construct_in_pass(
            quantized, theta, output_layout, batch * q_heads * q_blocks, k_blocks)
    else:
        # shapes outside the in-pass selection: the reference's route (capture workspace of 8
        # bytes per (query, key tile), block-mass kernel, library sort, stand-alone selector)
        workspace = torch.empty(capture_workspace_elements(quantized), dtype=torch.float32,
                                device=quantized.q.device)
        output = int8_attention_from_prequantized(quantized, output_layout=output_layout,
                                                  _block_mass=workspace)
        masses = workspace[: batch * q_heads * q_blocks * k_blocks].view(-1, k_blocks)
        row_offsets, block_indices, measured = select_retained_mass_csr(masses, theta)
    pattern = RetainedMassPattern(
        row_offsets=row_offsets, block_indices=block_indices, batch_size=batch, q_heads=q_heads,
        q_length=q_len, kv_length=quantized.k.shape[2], query_block_size=128,
        key_block_size=quantized.cta_k, attention_scale=quantized.attention_scale,
        retained_mass_target=float(theta), measured_retained_mass=measured,
        is_causal=quantized.is_causal, mask_signature=mask_signature(quantized.attn_mask),
        mask_reference=quantized.attn_mask)
    return output, pattern


@torch.inference_mode()
def construct_sparse_int8_attention(q, k, v, *, theta=0.99, scale=None, output_layout="hnd",
                                    v_quantization="absmax", is_causal=False, attn_mask=None):
    """Dense INT8 attention that also builds the reusable sparse support."""
    quantized = prequantize_int8_attention(q, k, v, scale=scale, v_quantization=v_quantization,
                                           is_causal=is_causal, attn_mask=attn_mask)
    return construct_sparse_int8_attention_from_prequantized(quantized, theta=theta,
                                                             output_layout=output_layout)


def sparse_int8_attention(q, k, v, sparse_pattern, *, scale=None, output_layout="hnd",
                          v_quantization="absmax", is_causal=False, attn_mask=None):
    """INT8 attention that visits only the key tiles of a frozen pattern; the pattern is built once
    (an early dense diffusion step) and reused on later, drifted inputs."""
    quantized = prequantize_int8_attention(q, k, v, scale=scale, v_quantization=v_quantization,
                                           is_causal=is_causal, attn_mask=attn_mask)
    return int8_attention_from_prequantized(quantized, sparse_pattern=sparse_pattern,
                                            output_layout=output_layout)
