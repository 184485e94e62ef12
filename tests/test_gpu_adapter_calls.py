"""The public API driven the way the reference's ComfyUI adapter drives it
(comfyui-risa-attention/node.py:44-71, 167-310): tensors arrive token-major as [B, N, H*D], are
viewed as [B, H, N, D] without a copy (so Q, K and V are strided), grouped-query K/V carry fewer
heads, masks arrive with two or three dimensions, and outputs are asked for in token-major storage
(``output_layout="nhd"``) so that the adapter's reshape back to [B, N, H*D] is free.  The adapter
itself is application glue over these calls; what is pinned here is the library's side of it."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import synthetic  # noqa: E402
from risaattention_b200._validation import apply_score_mask  # noqa: E402
from tests.util import nrmse  # noqa: E402


def _head_views(x, head_dim):
    """[B, N, H*D] -> [B, H, N, D] as a view (what the adapter does before every call)."""
    batch, tokens, width = x.shape
    return x.unsqueeze(3).reshape(batch, tokens, width // head_dim, head_dim).transpose(1, 2)


def _token_major(output, skip_output_reshape=False):
    """[B, H, N, D] -> [B, N, H*D] (the adapter's way back)."""
    if skip_output_reshape:
        return output
    batch, heads, tokens, head_dim = output.shape
    return output.transpose(1, 2).reshape(batch, tokens, heads * head_dim)


def _fp32(q, k, v, mask=None, scale=None):
    group = q.shape[1] // k.shape[1]
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    scores = q.float() @ k.float().repeat_interleave(group, 1).transpose(-1, -2) * scale
    if mask is not None:
        scores = apply_score_mask(scores, torch.broadcast_to(mask, scores.shape), False, 0)
    return scores.softmax(-1) @ v.float().repeat_interleave(group, 1)


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 8, 8), (128, 8, 2), (96, 6, 3)])
def test_dense_calls_on_token_major_tensors(head_dim, heads, kv_heads):
    g = torch.Generator(device="cuda").manual_seed(7)
    batch, tokens = 2, 1300
    flat_q = torch.randn(batch, tokens, heads * head_dim, device="cuda", generator=g).half()
    flat_k = torch.randn(batch, tokens, kv_heads * head_dim, device="cuda", generator=g).half()
    flat_v = torch.randn(batch, tokens, kv_heads * head_dim, device="cuda", generator=g).half()
    q, k, v = (_head_views(x, head_dim) for x in (flat_q, flat_k, flat_v))
    assert not q.is_contiguous() and q.data_ptr() == flat_q.data_ptr()
    want = _fp32(q, k, v, scale=0.11)

    # function form: one call, head-major result reshaped by the adapter
    direct = _token_major(risa.int8_attention(q, k, v, scale=0.11, attn_mask=None))
    assert direct.shape == flat_q.shape
    assert nrmse(_head_views(direct, head_dim), want) <= 0.03
    # the strides of the inputs do not change a bit of the result
    copies = risa.int8_attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=0.11)
    assert torch.equal(direct, _token_major(copies))

    # container form: quantise, drop the inputs, attend into token-major storage
    packed = risa.prequantize_int8_attention(q, k, v, scale=0.11, attn_mask=None)
    del q, k, v
    output = risa.int8_attention_from_prequantized(packed, output_layout="nhd")
    assert output.shape == (batch, heads, tokens, head_dim)
    flat = _token_major(output)
    if head_dim in (64, 128, 256):  # no channel padding: the adapter's reshape is a view
        assert output.transpose(1, 2).is_contiguous()
        assert flat.data_ptr() == output.data_ptr()
    assert torch.equal(flat, direct)
    # skip_output_reshape asks for head-major storage instead
    head_major = risa.int8_attention_from_prequantized(packed, output_layout="hnd")
    assert head_major.stride(1) > head_major.stride(2) and torch.equal(head_major, output)


@pytest.mark.parametrize("mask_dims", [2, 3])
def test_masks_of_two_and_three_dimensions(mask_dims):
    """The adapter pads a [Lq, Lk] or [B, Lq, Lk] mask with leading axes of size one and passes it
    on; boolean and additive forms, broadcast over heads (and batch)."""
    g = torch.Generator(device="cuda").manual_seed(11)
    batch, heads, tokens, head_dim = 2, 4, 300, 64
    q, k, v = (_head_views(torch.randn(batch, tokens, heads * head_dim, device="cuda",
                                       generator=g).half(), head_dim) for _ in range(3))
    keep = torch.rand(batch, tokens, tokens, device="cuda", generator=g) > 0.3
    keep[..., 0] = True  # no empty rows
    bias = torch.randn(batch, tokens, tokens, device="cuda", generator=g)
    for mask in (keep, bias):
        if mask_dims == 2:
            mask = mask[0].unsqueeze(0).unsqueeze(1)   # [Lq, Lk] -> [1, 1, Lq, Lk]
        else:
            mask = mask.unsqueeze(1)                   # [B, Lq, Lk] -> [B, 1, Lq, Lk]
        out = risa.int8_attention(q, k, v, scale=None, attn_mask=mask)
        assert nrmse(out, _fp32(q, k, v, mask)) <= 0.04
        packed = risa.prequantize_int8_attention(q, k, v, scale=None, attn_mask=mask)
        again = risa.int8_attention_from_prequantized(packed, output_layout="nhd")
        assert torch.equal(again, out)


def test_pattern_life_cycle_of_a_sampling_run():
    """First step of a sampling run: construct (dense output + frozen pattern).  Later steps, on
    drifted inputs: reuse, through either form of the call.  A pattern that keeps nearly everything
    is replaced by dense calls by the adapter (``sparsity`` below 0.05)."""
    batch, heads, kv_heads, tokens, head_dim = 1, 8, 2, 4096, 128
    q, k, v, g = synthetic.video_block_inputs(tokens, "cuda", seed=3, q_heads=heads,
                                              kv_heads=kv_heads, head_dim=head_dim, batch=batch)
    # token-major storage, as the adapter sees it
    q, k, v = (x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v))
    dense = risa.int8_attention(q, k, v, scale=None, attn_mask=None)

    built, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99, scale=None,
                                                          output_layout="nhd")
    assert built.transpose(1, 2).is_contiguous()
    assert nrmse(built, dense) <= 0.005  # construction returns the dense result
    assert 0.05 <= pattern.sparsity < 1.0 and pattern.measured_retained_mass >= 0.99 - 1e-6
    packed = risa.prequantize_int8_attention(q, k, v, scale=None, attn_mask=None)
    built_again, pattern_again = risa.construct_sparse_int8_attention_from_prequantized(
        packed, theta=0.99, output_layout="nhd")
    assert torch.equal(built_again, built)
    assert torch.equal(pattern_again.row_offsets, pattern.row_offsets)
    assert torch.equal(pattern_again.block_indices, pattern.block_indices)

    q2, k2, v2 = (synthetic.drift(x, g, "additive") for x in (q, k, v))
    reused = risa.sparse_int8_attention(q2, k2, v2, pattern, scale=None, output_layout="nhd")
    assert reused.transpose(1, 2).is_contiguous()
    packed2 = risa.prequantize_int8_attention(q2, k2, v2, scale=None, attn_mask=None)
    del q2, k2, v2
    through_packed = risa.int8_attention_from_prequantized(packed2, sparse_pattern=pattern,
                                                           output_layout="nhd")
    assert torch.equal(through_packed, reused)
    dense2 = risa.int8_attention_from_prequantized(packed2, sparse_pattern=None,
                                                   output_layout="nhd")
    # 99 % of the attention mass is kept: the sparse result stays close to the dense one
    assert nrmse(reused, dense2) <= 0.05
    flat = _token_major(reused)
    assert flat.shape == (batch, tokens, heads * head_dim) and flat.data_ptr() == reused.data_ptr()
