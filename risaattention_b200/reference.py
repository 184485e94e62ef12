"""FP32 retained-mass pattern construction and recall measurement: the evaluation tools of the
sparse path (reference src/risa_attention/reference.py:23-246).  Pure PyTorch on the caller's CUDA
device, chunked by 128 queries so the full attention matrix is never materialised."""
from __future__ import annotations

import math

import torch
from torch.nn import functional

from ._types import RetainedMassPattern
from ._validation import (SUPPORTED_DTYPES, apply_score_mask, is_available, kernel_head_dim,
                          mask_signature, select_key_block_size, validate_inputs)


def _block_masses(q, k, attn_mask, is_causal, scale, start, end, key_block, k_blocks):
    """[B, Hq, k_blocks] exact FP32 probability mass of the query rows start:end per key tile."""
    batch, q_heads, _, dim = q.shape
    kv_heads, k_len = k.shape[1], k.shape[2]
    grouped = q[:, :, start:end].reshape(batch, kv_heads, q_heads // kv_heads, end - start, dim)
    scores = torch.matmul(grouped.float(), k.float().transpose(-1, -2).unsqueeze(2)).mul_(scale)
    scores = apply_score_mask(scores.reshape(batch, q_heads, end - start, k_len), attn_mask,
                              is_causal, start)
    prob = torch.softmax(scores, dim=-1).nan_to_num_(nan=0.0)
    total = float(prob.sum())
    if k_len % key_block:
        prob = functional.pad(prob, (0, key_block - k_len % key_block))
    return prob.reshape(batch, q_heads, end - start, k_blocks, key_block).sum(dim=(2, 4)), total


@torch.inference_mode()
def build_retained_mass_pattern(q, k, *, theta=0.99, scale=None, attn_mask=None, is_causal=False):
    """Frozen retained-mass support from exact dense block masses (theta = retained-mass target)."""
    if not 0.0 < theta <= 1.0 or not math.isfinite(theta):
        raise ValueError("theta must be finite and in (0, 1]")
    if q.ndim != 4 or k.ndim != 4:
        raise ValueError("q and k must have shape [batch, heads, sequence, head_dim]")
    if q.dtype not in SUPPORTED_DTYPES or q.dtype != k.dtype:
        raise TypeError("q and k must have the same float32, float16, or bfloat16 dtype")
    if not q.is_cuda or q.device != k.device:
        raise ValueError("q and k must be on the same CUDA device")
    if not is_available(q.device):
        raise RuntimeError("sparse INT8 attention requires the CUDA extension and an SM100 GPU")
    batch, q_heads, q_len, dim = q.shape
    if k.shape[0] != batch or k.shape[3] != dim:
        raise ValueError("sparse attention requires self-attention with equal Q/K lengths")
    attn_mask = validate_inputs(q, k, k, attn_mask)
    k_len = k.shape[2]
    attention_scale = dim ** -0.5 if scale is None else float(scale)
    if not math.isfinite(attention_scale):
        raise ValueError("scale must be finite")
    key_block = select_key_block_size(
        kernel_head_dim(dim), k_len, has_mask=attn_mask is not None and attn_mask.stride(-2) != 0)
    q_blocks, k_blocks = math.ceil(q_len / 128), math.ceil(k_len / key_block)
    keep = torch.zeros(batch, q_heads, q_blocks, k_blocks, dtype=torch.bool, device=q.device)
    retained = torch.zeros((), dtype=torch.float64, device=q.device)
    total = torch.zeros((), dtype=torch.float64, device=q.device)
    for block in range(q_blocks):
        masses, _ = _block_masses(q, k, attn_mask, is_causal, attention_scale, block * 128,
                                  min(q_len, block * 128 + 128), key_block, k_blocks)
        ordered, order = masses.sort(dim=-1, descending=True)
        target = theta * masses.sum(dim=-1, keepdim=True)
        counts = ((ordered.cumsum(dim=-1) < target).sum(dim=-1) + 1).clamp_(max=k_blocks)
        chosen = torch.arange(k_blocks, device=q.device) < counts[..., None]
        keep[:, :, block].scatter_(-1, order, chosen)
        retained += (masses * keep[:, :, block]).sum().double()
        total += masses.sum().double()
    flat = keep.reshape(-1, k_blocks)
    if not bool(flat.any(dim=-1).all()):
        raise RuntimeError("retained-mass construction produced an empty support row")
    row_offsets = torch.zeros(flat.shape[0] + 1, dtype=torch.int32, device=q.device)
    row_offsets[1:] = flat.sum(dim=-1).cumsum(0)
    block_indices = flat.nonzero()[:, 1].to(torch.int32).contiguous()
    return RetainedMassPattern(
        row_offsets=row_offsets, block_indices=block_indices, batch_size=batch, q_heads=q_heads,
        q_length=q_len, kv_length=k_len, query_block_size=128, key_block_size=key_block,
        attention_scale=attention_scale, retained_mass_target=float(theta),
        measured_retained_mass=float(retained) / max(float(total), 1e-20), is_causal=is_causal,
        mask_signature=mask_signature(attn_mask), mask_reference=attn_mask)


@torch.inference_mode()
def measure_pattern_recall(q, k, sparse_pattern, *, attn_mask=None) -> float:
    """Exact dense attention mass that a frozen pattern retains."""
    if not isinstance(sparse_pattern, RetainedMassPattern):
        raise TypeError("sparse_pattern must be returned by build_retained_mass_pattern")
    if q.ndim != 4 or k.ndim != 4 or q.device != k.device or not q.is_cuda:
        raise ValueError("q and k must be 4D tensors on the same CUDA device")
    attn_mask = validate_inputs(q, k, k, attn_mask)
    if mask_signature(attn_mask) != sparse_pattern.mask_signature:
        raise ValueError("pattern mask has changed")
    batch, q_heads, q_len, dim = q.shape
    kv_heads, k_len = k.shape[1], k.shape[2]
    if k.shape != (batch, kv_heads, k_len, dim) or q.dtype != k.dtype or q_heads % kv_heads:
        raise ValueError("q and k shapes/dtypes are incompatible")
    if (batch, q_heads, q_len, k_len) != (sparse_pattern.batch_size, sparse_pattern.q_heads,
                                          sparse_pattern.q_length, sparse_pattern.kv_length):
        raise ValueError("q and k do not match the frozen retained-mass pattern")
    if sparse_pattern.row_offsets.device != q.device:
        raise ValueError("pattern and q/k must be on the same CUDA device")
    key_block = sparse_pattern.key_block_size
    q_blocks, k_blocks = math.ceil(q_len / 128), math.ceil(k_len / key_block)
    rows = batch * q_heads * q_blocks
    counts = sparse_pattern.row_offsets[1:] - sparse_pattern.row_offsets[:-1]
    row_of = torch.repeat_interleave(torch.arange(rows, device=q.device), counts.long())
    keep = torch.zeros(rows, k_blocks, dtype=torch.bool, device=q.device)
    keep[row_of, sparse_pattern.block_indices.long()] = True
    keep = keep.reshape(batch, q_heads, q_blocks, k_blocks)
    retained, total = 0.0, 0.0
    for block in range(q_blocks):
        masses, mass = _block_masses(q, k, attn_mask, sparse_pattern.is_causal,
                                     sparse_pattern.attention_scale, block * 128,
                                     min(q_len, block * 128 + 128), key_block, k_blocks)
        retained += float((masses * keep[:, :, block]).sum())
        total += mass
    return retained / max(total, 1e-20)
