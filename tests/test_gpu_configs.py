"""Scaled-down versions of the benchmark configurations that are not the headline bench line:
the video-DiT-shaped self-attention (sequence length not a multiple of 128, per-channel spread,
outlier channels; dense, pattern construction and sparse reuse) and the edge / feature sweep
(head_dim 64 and 256, Lq != Lk, causal, additive and boolean masks with fully masked rows,
batch 2, LSE, prequantise -> attend).  Everything is compared with the reference's own kernels on
the same inputs: codes and tile sets bit for bit, outputs within 2e-3 x RMS (+ 1 ulp of bf16)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from tests.util import assert_outputs_match  # noqa: E402

TOL = 2e-3


def _video_inputs(heads, length, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)

    def make():
        x = torch.randn(1, heads, length, 128, device="cuda", generator=g)
        std = torch.empty(128, device="cuda").uniform_(0.5, 2.0, generator=g)
        outliers = torch.randperm(128, device="cuda", generator=g)[:2]  # ~1 % of the channels
        std[outliers] *= 20.0
        return (x * std).bfloat16()

    return make(), make(), make()


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_video_dit_shape_dense_and_sparse(ref, mode):
    heads, length = 5, 2040  # 15 full 128-token blocks and one of 120, like 32760 = 255 * 128 + 120
    q, k, v = _video_inputs(heads, length)
    affine = mode == "midpoint_affine"
    want_pk = ref.prequantize(q, k, v, cta_k=128, midpoint_affine=affine)
    pk = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
    assert pk.cta_k == 128
    for name, ours in (("q", pk.q), ("k", pk.k), ("v", pk.v), ("q_scale", pk.q_scale),
                       ("k_scale", pk.k_scale), ("v_scale", pk.v_scale)):
        assert torch.equal(ours.reshape(-1), want_pk[name].reshape(-1)), name
    want = ref.attention(want_pk, sm_scale=128 ** -0.5)
    got = risa.int8_attention(q, k, v, v_quantization=mode)
    assert_outputs_match(got, want["out"], TOL)

    out, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99, v_quantization=mode)
    cap = ref.attention(want_pk, sm_scale=128 ** -0.5, capture=True)
    n_q = n_k = 16
    masses = cap["workspace"][: heads * n_q * n_k].view(-1, n_k)
    rro, rbi, _ = ref.select_retained_mass(masses, 0.99)
    assert torch.equal(pattern.row_offsets, rro) and torch.equal(pattern.block_indices, rbi)
    assert_outputs_match(out, cap["out"], TOL)
    reuse = risa.sparse_int8_attention(q, k, v, pattern, v_quantization=mode)
    if pattern.sparsity < 0.05:
        # a nearly dense support runs the dense kernel, as in the reference (_execution.py:227-228)
        assert_outputs_match(reuse, want["out"], TOL)
    else:
        want_s = ref.attention(want_pk, sm_scale=128 ** -0.5, row_offsets=rro, block_indices=rbi)
        assert_outputs_match(reuse, want_s["out"], TOL)
    # the sparse kernel itself, on the same tile lists, whatever the sparsity
    from tests.test_gpu_attention import _ours
    got_s = _ours(want_pk, sm_scale=128 ** -0.5, path=0, row_offsets=rro, block_indices=rbi)
    want_s = ref.attention(want_pk, sm_scale=128 ** -0.5, row_offsets=rro, block_indices=rbi)
    assert_outputs_match(got_s["out"], want_s["out"], TOL)


@pytest.mark.parametrize("dim", [64, 256])
@pytest.mark.parametrize("mask_kind", ["causal", "bias", "bool_rows"])
def test_edge_sweep(ref, dim, mask_kind):
    b, hq, hkv, lq, lk = 2, 8, 2, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(dim)
    q = torch.randn(b, hq, lq, dim, device="cuda", generator=g).bfloat16()
    k = torch.randn(b, hkv, lk, dim, device="cuda", generator=g).bfloat16()
    v = torch.randn(b, hkv, lk, dim, device="cuda", generator=g).bfloat16()
    mask, causal = None, False
    if mask_kind == "causal":
        causal = True
    elif mask_kind == "bias":
        mask = torch.randn(b, hq, lq, lk, device="cuda", generator=g)
    else:
        mask = torch.ones(b, hq, lq, lk, device="cuda", dtype=torch.bool)
        dead = torch.randperm(lq, device="cuda", generator=g)[: lq // 10]
        mask[:, :, dead] = False
    pk = risa.prequantize_int8_attention(q, k, v, attn_mask=mask, is_causal=causal,
                                         return_lse=True)
    out, lse = risa.int8_attention_from_prequantized(pk, return_lse=True)
    direct, lse_direct = risa.int8_attention(q, k, v, attn_mask=mask, is_causal=causal,
                                             return_lse=True)
    assert torch.equal(out, direct) and torch.equal(lse, lse_direct)

    cta_k = pk.cta_k
    assert cta_k == (64 if (mask is not None or dim == 64) else 128)
    want_pk = ref.prequantize(q, k, v, cta_k=cta_k)
    assert torch.equal(pk.q, want_pk["q"]) and torch.equal(pk.k, want_pk["k"])
    assert torch.equal(pk.v.reshape(-1), want_pk["v"].reshape(-1))
    full_mask = None if mask is None else mask.expand(b, hq, lq, lk)
    want = ref.attention(want_pk, sm_scale=dim ** -0.5, mask=full_mask, is_causal=causal,
                         want_lse=True)
    assert_outputs_match(out, want["out"], TOL)
    want_lse = want["lse"] + ref.lse_shift(q, k, want_pk["anchors"], dim ** -0.5)
    assert torch.equal(torch.isneginf(lse), torch.isneginf(want_lse))
    fin = torch.isfinite(want_lse)
    torch.testing.assert_close(lse[fin], want_lse[fin], rtol=0, atol=5e-4)
    if mask_kind == "bool_rows":
        assert torch.count_nonzero(out[:, :, dead]) == 0
        assert torch.isneginf(lse[:, :, dead]).all()
