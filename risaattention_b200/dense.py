"""Public dense attention call and its torch.library operators
(reference src/risa_attention/dense.py:14-146; operator names and schemas are kept so compiled
graphs written against the reference resolve)."""
from __future__ import annotations

import torch

from ._execution import execute_dense_attention, int8_attention_from_prequantized
from ._quantization import prequantize_int8_attention
from ._validation import uses_centered_values


def _op_int8_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None,
                       use_midpoint_affine: bool, is_causal: bool) -> torch.Tensor:
    return execute_dense_attention(q, k, v, scale=scale, attn_mask=None,
                                   use_midpoint_affine=use_midpoint_affine, is_causal=is_causal)


def _fake_int8_attention(q, k, v, scale, use_midpoint_affine, is_causal):
    return q.new_empty(q.shape)


def _op_int8_attention_masked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                              attn_mask: torch.Tensor, scale: float | None,
                              use_midpoint_affine: bool, is_causal: bool) -> torch.Tensor:
    return execute_dense_attention(q, k, v, scale=scale, attn_mask=attn_mask,
                                   use_midpoint_affine=use_midpoint_affine, is_causal=is_causal)


def _fake_int8_attention_masked(q, k, v, attn_mask, scale, use_midpoint_affine, is_causal):
    return q.new_empty(q.shape)


def _register(name, implementation, fake) -> bool:
    """Defines ``risa_attention::<name>`` with the reference's schema unless the process already
    has it (the reference package imported side by side registers the same names; a second
    definition is an error, and its operators then stay in charge of compiled graphs)."""
    try:
        operator = torch.library.custom_op(f"risa_attention::{name}", mutates_args=())(
            implementation)
    except RuntimeError:
        return False
    operator.register_fake(fake)
    return True


OPERATORS_REGISTERED = (
    _register("int8_attention", _op_int8_attention, _fake_int8_attention),
    _register("int8_attention_masked", _op_int8_attention_masked, _fake_int8_attention_masked),
)


def int8_attention(q, k, v, *, scale=None, attn_mask=None, v_quantization="absmax",
                   is_causal=False, return_lse=False, kv_permutation=None, fuse_gather=True):
    """Inference SDPA with signed INT8 Q/K/V and unsigned INT8 probabilities.

    Layout ``[batch, heads, sequence, head_dim]``; grouped-query attention and unequal Q/K lengths
    are supported; head dims are padded to 64/128/256 and sliced back.  Q and K get the same block
    Hadamard rotation (H4 for up to 256 keys, H64 for D64, signed H128 for D128, plain H128 per
    half for D256) before symmetric INT8 quantisation, K optionally translated by a sampled anchor
    key (softmax-invariant).  V is quantised per channel (absmax, or midpoint_affine with a
    residual-corrected centre).  Scores, maxima, exponentials, denominators and V dequantisation
    are FP32; the denominator uses the same rounded U8 probabilities as P*V."""
    if return_lse or kv_permutation is not None:
        packed = prequantize_int8_attention(
            q, k, v, scale=scale, attn_mask=attn_mask, v_quantization=v_quantization,
            is_causal=is_causal, return_lse=return_lse, kv_permutation=kv_permutation,
            fuse_gather=fuse_gather)
        return int8_attention_from_prequantized(packed, return_lse=return_lse)
    affine = uses_centered_values(v_quantization)
    if not torch.compiler.is_compiling() and type(q) is torch.Tensor:
        # eager call on plain tensors: same implementation as the registered operators, without
        # the dispatcher's per-call cost (traced / compiled graphs and tensor subclasses such as
        # fake tensors go through the operators and their shape-only implementations)
        return execute_dense_attention(q, k, v, scale=scale, attn_mask=attn_mask,
                                       use_midpoint_affine=affine, is_causal=is_causal)
    if attn_mask is None:
        return torch.ops.risa_attention.int8_attention(q, k, v, scale, affine, is_causal)
    return torch.ops.risa_attention.int8_attention_masked(q, k, v, attn_mask, scale, affine,
                                                          is_causal)
