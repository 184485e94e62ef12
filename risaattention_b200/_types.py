"""Packed operands and frozen sparse support, field-for-field as in the reference
(src/risa_attention/_types.py:13-79) so objects can be exchanged with code written against it."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True, slots=True)
class PrequantizedInt8Attention:
    """INT8 Q/K/V codes, their scales, V centres and launch metadata.

    Produced by :func:`prequantize_int8_attention`; holds no floating-point Q, K or V."""

    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    q_scale: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    v_center: torch.Tensor
    original_head_dim: int
    input_dtype: torch.dtype
    attention_scale: float
    cta_k: int
    attn_mask: torch.Tensor | None
    v_quantization: str = "absmax"
    is_causal: bool = False
    lse_shift: torch.Tensor | None = None
    kv_permuted: bool = False


@dataclass(frozen=True, slots=True)
class RetainedMassPattern:
    """Per-head block support in CSR form on the GPU.

    Rows are ordered ``[batch, query_head, query_block]``; each row lists ascending key-tile ids."""

    row_offsets: torch.Tensor
    block_indices: torch.Tensor
    batch_size: int
    q_heads: int
    q_length: int
    kv_length: int
    query_block_size: int
    key_block_size: int
    attention_scale: float
    retained_mass_target: float
    measured_retained_mass: float
    is_causal: bool = False
    mask_signature: tuple | None = None
    mask_reference: torch.Tensor | None = None

    @property
    def coverage(self) -> float:
        rows = self.batch_size * self.q_heads * math.ceil(self.q_length / self.query_block_size)
        return self.block_indices.numel() / (rows * math.ceil(self.kv_length / self.key_block_size))

    @property
    def sparsity(self) -> float:
        return 1.0 - self.coverage

    @property
    def index_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.row_offsets, self.block_indices))
