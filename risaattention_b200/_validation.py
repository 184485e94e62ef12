"""Input contracts, mask semantics and key-tile selection
(reference src/risa_attention/_validation.py:11-148)."""
from __future__ import annotations

import torch

from . import _backend

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
KEY_BLOCK_SIZE = 64
LARGE_KEY_BLOCK_SIZE = 128
SUPPORTED_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
MIN_PATTERN_SPARSITY = 0.05
OUTPUT_LAYOUTS = ("hnd", "nhd")
VALUE_QUANTIZATION_MODES = ("midpoint_affine", "absmax")
UNAVAILABLE = "INT8 attention requires the risa_attention CUDA extension and an NVIDIA SM100 GPU"


def uses_centered_values(v_quantization: str) -> bool:
    if v_quantization not in VALUE_QUANTIZATION_MODES:
        raise ValueError(
            f"v_quantization must be one of {VALUE_QUANTIZATION_MODES}, got {v_quantization!r}")
    return v_quantization == "midpoint_affine"


def mask_signature(mask: torch.Tensor | None) -> tuple | None:
    """Identity of a mask tensor; a retained pattern is only valid for the mask it was built with."""
    if mask is None:
        return None
    try:
        version = mask._version
    except RuntimeError:  # inference tensors carry no version counter
        version = None
    return (mask.data_ptr(), version, tuple(mask.shape), tuple(mask.stride()), mask.dtype, mask.device)


def apply_score_mask(scores, attn_mask, is_causal, start):
    """FP32 specification of mask and causal handling for rows ``start:start+rows`` of the scores.
    Causal masking is aligned to the upper-left corner."""
    rows = scores.shape[-2]
    if attn_mask is not None:
        window = attn_mask[..., start:start + rows, :]
        scores = scores.masked_fill(~window, -torch.inf) if window.dtype == torch.bool else scores + window
    if is_causal:
        q_idx = torch.arange(start, start + rows, device=scores.device)[:, None]
        k_idx = torch.arange(scores.shape[-1], device=scores.device)[None, :]
        scores = scores.masked_fill(k_idx > q_idx, -torch.inf)
    return scores


def pad_key_length(length: int, key_block_size: int = KEY_BLOCK_SIZE) -> int:
    return -(-length // key_block_size) * key_block_size


def kernel_head_dim(head_dim: int) -> int:
    return 64 if head_dim <= 64 else 128 if head_dim <= 128 else 256


def select_key_block_size(kernel_head_dim: int, key_length: int, *, has_mask: bool) -> int:
    """128-key tiles need no per-query mask, a head dim of at least 128 and more than 1024 keys."""
    if not has_mask and kernel_head_dim >= 128 and key_length > 1024:
        return LARGE_KEY_BLOCK_SIZE
    return KEY_BLOCK_SIZE


def is_available(device: torch.device | int | None = None) -> bool:
    return _backend.is_available(device)


def validate_inputs(q, k, v, attn_mask):
    """Checks the public tensor contract and returns the mask expanded to [B, Hq, Lq, Lk]."""
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape [batch, heads, sequence, head_dim]")
    if q.dtype not in SUPPORTED_DTYPES:
        raise TypeError(f"q, k, and v must be float32, float16, or bfloat16, got {q.dtype}")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(
            f"q, k, and v must have the same dtype, got {q.dtype}, {k.dtype}, and {v.dtype}")
    if not q.is_cuda or q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must be on the same CUDA device")
    if not is_available(q.device):
        raise RuntimeError(UNAVAILABLE)
    batch, q_heads, q_len, head_dim = q.shape
    k_batch, kv_heads, k_len, k_dim = k.shape
    if v.shape != (batch, kv_heads, k_len, head_dim):
        raise ValueError(
            f"v must have shape [q.batch, k.heads, k.sequence, q.head_dim], got {tuple(v.shape)}")
    if k_batch != batch or k_dim != head_dim:
        raise ValueError(
            f"q and k batch/head dimensions must match, got {tuple(q.shape)} and {tuple(k.shape)}")
    if min(batch, q_heads, kv_heads, q_len, k_len) == 0:
        raise ValueError("batch, head counts, and sequence lengths must be positive")
    if q_heads % kv_heads:
        raise ValueError(
            f"q head count ({q_heads}) must be divisible by k/v head count ({kv_heads})")
    if not 0 < head_dim <= 256:
        raise ValueError(f"head_dim must be in [1, 256], got {head_dim}")
    if q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1:
        raise ValueError("the last dimension of q, k, and v must be contiguous")
    if attn_mask is None:
        return None
    if attn_mask.device != q.device:
        raise ValueError("attn_mask must be on the same CUDA device as q, k, and v")
    if attn_mask.dtype not in (torch.bool, torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("attn_mask must be bool, float16, bfloat16, or float32")
    try:
        return torch.broadcast_to(attn_mask, (batch, q_heads, q_len, k_len))
    except RuntimeError as error:
        raise ValueError(
            f"attn_mask must be broadcastable to [{batch}, {q_heads}, {q_len}, {k_len}], "
            f"got {tuple(attn_mask.shape)}") from error
