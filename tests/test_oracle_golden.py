"""Pins the CPU oracle on the known-answer cases of the reference's own tests (pure-integer or
power-of-two data, where no approximate GPU instruction can matter) and on the committed golden
fixtures produced by the reference kernels on a B200."""
import json
from pathlib import Path

import pytest
import torch

from oracle import risa_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("length", [1025, 2049])
def test_v_absmax_known_answer(dtype, length):
    """reference tests/cuda/test_value_quantization.py:18-52."""
    batch, heads, channels = 2, 3, 128
    tokens = torch.arange(length)[None, None, :, None]
    offs = torch.arange(batch * heads).reshape(batch, heads, 1, 1)
    codes = ((tokens + offs) % 255 - 127).expand(batch, heads, length, channels)
    scales = 2.0 ** ((torch.arange(channels) % 4).float() - 2)
    v = (codes * scales).to(dtype)
    packed, sc, center = O.quantize_v(v.float(), 128, False)
    padded = packed.shape[-1]
    expected = torch.zeros(batch, heads, channels, padded, dtype=torch.int8)
    expected[..., :length] = codes.transpose(2, 3).to(torch.int8)
    order = torch.tensor([0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15])
    expected = expected.reshape(batch, heads, channels, -1, 16)[..., order]
    assert torch.equal(packed.reshape_as(expected), expected)
    assert torch.equal(sc.reshape(batch, heads, channels), scales.expand(batch, heads, channels))
    assert torch.count_nonzero(center) == 0


@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("length", [65, 193])
def test_capture_tile_max_known_answer(dim, length):
    """reference tests/cuda/test_risa_attention.py:20-79: hand-filled packed operands."""
    lq, hq = 137, 2
    cta_k = 64
    blocks = -(-length // cta_k)
    q = torch.ones(1, hq, lq, dim, dtype=torch.int8)
    k = torch.zeros(1, 1, length, dim, dtype=torch.int8)
    for i in range(blocks):
        k[:, :, i * cta_k:(i + 1) * cta_k] = 3 if i % 2 == 0 else -2
    vq, vs, vc = O.quantize_v(torch.randn(1, 1, length, dim) + 2, cta_k, False)
    qs = torch.ones(1, hq, -(-lq // 128) * (64 if dim == 256 else 32))
    ks = torch.ones(1, 1, blocks * 4)
    plain = O.attention(q, k, vq, qs, ks, vs, vc, cta_k=cta_k, sm_scale=1 / 128,
                        out_dtype=torch.float16)
    cap = O.attention(q, k, vq, qs, ks, vs, vc, cta_k=cta_k, sm_scale=1 / 128, capture=True,
                      out_dtype=torch.float16)
    assert torch.equal(plain["out"], cap["out"])
    rows = hq * lq
    mass_elements = hq * 2 * blocks
    if blocks > 1:
        maxima = cap["workspace"][mass_elements:mass_elements + rows * (blocks - 1) * 2]
        maxima = maxima.reshape(rows, blocks - 1, 2)[..., 1]
        levels = torch.tensor([3 if i % 2 == 0 else -2 for i in range(blocks)])
        scale = torch.tensor(1.44269504088896340736) / 128
        expected = (levels[:-1].double() * dim * scale.double()
                    - torch.tensor(7.9943534).double()).float()
        assert torch.equal(maxima, expected.expand_as(maxima))
    hidden = torch.zeros(1, hq, lq, length, dtype=torch.bool)
    empty = O.attention(q, k, vq, qs, ks, vs, vc, cta_k=cta_k, sm_scale=1 / 128, mask=hidden,
                        out_dtype=torch.float16)
    assert torch.count_nonzero(empty["out"]) == 0


@pytest.mark.parametrize("scale", [None, 0.0, -0.125])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_constant_values_preserve_probability_mass(scale, mode):
    """reference tests/cuda/test_probability_mass.py:21-34."""
    torch.manual_seed(41)
    q = torch.randn(1, 2, 70, 64).bfloat16()
    k = torch.randn(1, 1, 300, 64).bfloat16()
    values = torch.linspace(-3, 5, 64).bfloat16()
    v = values.expand_as(k).contiguous()
    out = O.int8_attention(q, k, v, scale=scale, v_quantization=mode)
    assert torch.equal(out, values.expand_as(out))


def test_masked_rows_and_lse_at_zero_scale():
    """reference tests/cuda/test_probability_mass.py:37-70."""
    torch.manual_seed(43)
    lk = 300
    q = torch.randn(1, 2, 67, 64).bfloat16()
    k = torch.randn(1, 1, lk, 64).bfloat16()
    v = torch.full_like(k, 3)
    mask = torch.ones(67, lk, dtype=torch.bool)
    mask[0] = False
    mask[1:, 7::9] = False
    out, lse = O.int8_attention(q, k, v, scale=0.0, attn_mask=mask, is_causal=True, return_lse=True)
    assert torch.equal(out[:, :, 1:], torch.full_like(out[:, :, 1:], 3))
    assert torch.count_nonzero(out[:, :, 0]) == 0 and torch.isneginf(lse[:, :, 0]).all()
    visible = mask & (torch.arange(lk)[None, :] <= torch.arange(67)[:, None])
    torch.testing.assert_close(lse, visible.sum(-1).float().log().expand_as(lse), atol=2e-5, rtol=0)


def test_key_mask_tiles_known_answer():
    """reference tests/cuda/test_key_mask_tiles.py:79-103: tiles [4..9], count 6."""
    mask = torch.ones(1, 4, 1, 1153, dtype=torch.bool)
    mask[..., :512] = False
    tiles = O.key_mask_tiles(mask.expand(1, 4, 257, 1153), 128)
    assert torch.equal(tiles[..., :6], torch.tensor([4, 5, 6, 7, 8, 9], dtype=torch.int32).expand(1, 4, 6))
    assert (tiles[..., -1] == 6).all()


def test_lse_shift_formula():
    """reference tests/cuda/test_lse_correction.py:9-31."""
    torch.manual_seed(35)
    q = torch.randn(2, 4, 17, 64)
    k = torch.randn(2, 2, 9, 64)
    anchors = torch.tensor([[-1, 0], [3, 2]], dtype=torch.int32)
    out = O.lse_shift(q, k, anchors, 64 ** -0.5)
    sel = k.gather(2, anchors.clamp_min(0).long()[..., None, None].expand(2, 2, 1, 64))
    sel = sel * (anchors >= 0)[..., None, None]
    want = (q * sel.repeat_interleave(2, 1)).sum(-1) * 64 ** -0.5
    torch.testing.assert_close(out, want, rtol=2e-5, atol=5e-6)
    assert torch.count_nonzero(out[0, :2]) == 0


def test_accuracy_against_fp32_sdpa():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 4, 256, 128), torch.randn(1, 1, 1024, 128), torch.randn(1, 1, 1024, 128)
    out, lse = O.int8_attention(q, k, v, return_lse=True)
    want, want_lse = O.sdpa_fp32(q, k, v)
    err = ((out.float() - want).pow(2).mean() / want.pow(2).mean()).sqrt()
    assert err < 0.017
    torch.testing.assert_close(lse, want_lse, atol=0.02, rtol=0)


def test_golden_fixtures_from_reference_kernels():
    """Codes, scales, anchors, capture statistics and tile sets that the reference's own kernels
    produced on a B200 (tests/golden/make_golden.py); the CPU oracle must reproduce them within its
    documented budget (approximate GPU division / exp2 cannot be matched bit for bit on a CPU)."""
    path = GOLDEN / "reference_b200.pt"
    if not path.exists():
        pytest.skip("golden fixtures not generated yet")
    gold = torch.load(path)
    for case in gold["cases"]:
        g = torch.Generator().manual_seed(case["seed"])
        b, hq, hkv, lq, lk, d = case["shape"]
        q = torch.randn(b, hq, lq, d, generator=g).bfloat16()
        k = torch.randn(b, hkv, lk, d, generator=g).bfloat16()
        v = torch.randn(b, hkv, lk, d, generator=g).bfloat16()
        if case["anchor"]:
            k = (k.float() * 0.1 + 4).bfloat16()
        anchors = O.detect_k_anchor(k.float())
        assert torch.equal(anchors, case["anchors"])
        qc, qs = O.quantize_q(q.float(), lk)
        kc, ks = O.quantize_k(k.float(), case["cta_k"], anchors)
        vc, vs, vcen = O.quantize_v(v.float(), case["cta_k"], case["affine"])
        for mine, ref in ((qc, case["q"]), (kc, case["k"]), (vc, case["v"])):
            diff = (mine.int() - ref.int()).abs()
            assert diff.max() <= 1 and (diff > 0).float().mean() < 2e-3
        torch.testing.assert_close(qs, case["q_scale"], rtol=1e-6, atol=0)
        torch.testing.assert_close(ks, case["k_scale"], rtol=1e-6, atol=0)
        torch.testing.assert_close(vs, case["v_scale"], rtol=1e-6, atol=0)
        r = O.attention(case["q"], case["k"], case["v"], case["q_scale"], case["k_scale"],
                        case["v_scale"], case["v_center"], cta_k=case["cta_k"],
                        sm_scale=d ** -0.5, capture=True, want_lse=True)
        rms = case["out"].float().pow(2).mean().sqrt()
        assert ((r["out"].float() - case["out"].float()).abs().max() / rms) < 2e-3 + 2 ** -7 * 4
        n_mass = case["masses"].numel()
        torch.testing.assert_close(r["workspace"][:n_mass].view_as(case["masses"]), case["masses"],
                                   rtol=2e-3, atol=2e-3)
        ro, bi, _ = O.select_retained_mass(case["masses"], case["theta"])
        assert torch.equal(ro, case["row_offsets"]) and torch.equal(bi, case["block_indices"])
