"""Fused attention kernels against the reference's own kernels on identical packed operands:
capture statistics, block masses and tile sets bit for bit; outputs and LSE within
2e-3 x RMS(output) (the row kernel keeps the reference's FP32 operation order, so it is also
required to match bit for bit)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.util import assert_outputs_match, nrmse, qkv, rel_max_err  # noqa: E402

TOL = 2e-3  # max |ours - reference| / RMS(reference output)


def _packed(ref, d, lq, lk, hq, hkv, cta_k, dtype=torch.bfloat16, affine=False, seed=0, b=1):
    q, k, v = qkv(b, hq, hkv, lq, lk, d, dtype, seed=seed)
    v = v + 0.5
    pk = ref.prequantize(q, k, v, cta_k=cta_k, midpoint_affine=affine)
    return q, k, v, pk


def _ours(pk, *, sm_scale, path, out_dtype=torch.bfloat16, mask=None, is_causal=False,
          row_offsets=None, block_indices=None, capture=False, want_lse=False, tiles=None):
    from risaattention_b200 import _backend

    q, k = pk["q"], pk["k"]
    b, hq, lq, d = q.shape
    lk, cta_k = k.shape[2], pk["cta_k"]
    out = torch.empty(b, hq, lq, d, dtype=out_dtype, device=q.device)
    lse = torch.empty(b, hq, lq, device=q.device) if want_lse else None
    ws = None
    if capture:
        n_q, n_k = -(-lq // 128), -(-lk // cta_k)
        ws = torch.empty(b * hq * n_q * n_k + b * hq * lq * (2 * n_k + 2), device=q.device)
    prev = _backend._C.set_attention_path(path)
    try:
        _backend._C.risa_sdpa_prequantized(
            q, k, pk["v"], out, pk["q_scale"], pk["k_scale"], pk["v_scale"], pk["v_center"],
            cta_k, sm_scale, 1 if out_dtype == torch.float16 else 2,
            torch.cuda.current_stream().cuda_stream, attn_mask=mask,
            sparse_row_offsets=row_offsets, sparse_block_indices=block_indices, block_mass=ws,
            is_causal=is_causal, lse=lse, key_mask_tiles=tiles)
    finally:
        _backend._C.set_attention_path(prev)
    torch.cuda.synchronize()
    return {"out": out, "lse": lse, "workspace": ws}


SHAPES = [
    # d, lq, lk, hq, hkv, cta_k
    (64, 137, 263, 2, 1, 64),
    (128, 137, 263, 2, 1, 64),
    (128, 300, 1153, 4, 2, 128),
    (256, 137, 263, 2, 1, 64),
    (256, 130, 1100, 2, 2, 128),
]


def _masks(kind, b, hq, lq, lk):
    if kind == "none":
        return None
    if kind == "key_bias":
        return torch.linspace(-2, 0, lk, device="cuda")[None, None, None, :].expand(b, hq, lq, lk)
    if kind == "row_bool":
        m = torch.ones(lq, lk, device="cuda", dtype=torch.bool)
        m[0] = False
        m[1:, 7::9] = False
        return m[None, None].expand(b, hq, lq, lk)
    if kind == "bias_4d":
        g = torch.Generator(device="cuda").manual_seed(11)
        return torch.randn(b, hq, lq, lk, device="cuda", generator=g)
    raise ValueError(kind)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("mask_kind", ["none", "key_bias", "row_bool", "bias_4d"])
@pytest.mark.parametrize("causal", [False, True])
def test_row_kernel_matches_reference(ref, shape, mask_kind, causal):
    d, lq, lk, hq, hkv, cta_k = shape
    if mask_kind in ("row_bool", "bias_4d") and cta_k == 128:
        pytest.skip("per-query masks always use 64-key tiles")
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, affine=True, seed=d + lk)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    for scale in (d ** -0.5, 0.0, -0.125):
        want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, want_lse=True)
        assert_outputs_match(got["out"], want["out"], TOL)
        if mask_kind == "none":
            # same FP32 operation order as the reference: bit-identical without a mask
            assert torch.equal(got["out"], want["out"])
        assert torch.equal(torch.isneginf(got["lse"]), torch.isneginf(want["lse"]))
        fin = torch.isfinite(want["lse"])
        torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0, atol=2e-4)
        if mask_kind == "row_bool":
            assert torch.count_nonzero(got["out"][:, :, 0]) == 0
            assert torch.isneginf(got["lse"][:, :, 0]).all()


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("mask_kind", ["none", "key_bias"])
def test_capture_and_selection_bit_exact(ref, shape, causal, mask_kind):
    from risaattention_b200.sparse import select_retained_mass_csr

    d, lq, lk, hq, hkv, cta_k = shape
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, seed=7 + d)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    scale = d ** -0.5
    want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, capture=True)
    got = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, capture=True)
    n_q, n_k = -(-lq // 128), -(-lk // cta_k)
    if mask_kind == "none":
        assert torch.equal(got["workspace"].view(torch.int32), want["workspace"].view(torch.int32))
        assert torch.equal(got["out"], want["out"])
    else:
        # masked scores may differ from the reference in the last FP32 bit (see apply_mask)
        torch.testing.assert_close(got["workspace"][: hq * n_q * n_k],
                                   want["workspace"][: hq * n_q * n_k], rtol=1e-4, atol=1e-5)
        assert_outputs_match(got["out"], want["out"], TOL)
    masses = got["workspace"][: hq * n_q * n_k].view(-1, n_k)
    for theta in (0.5, 0.99, 1.0):
        ro, bi, mm = select_retained_mass_csr(masses, theta)
        rro, rbi, rmm = ref.select_retained_mass(masses, theta)
        assert torch.equal(ro, rro) and torch.equal(bi, rbi) and mm == rmm
        # sparse reuse over the selected tiles
        want_s = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, row_offsets=rro,
                               block_indices=rbi)
        got_s = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, row_offsets=ro,
                      block_indices=bi)
        if mask_kind == "none":
            assert torch.equal(got_s["out"], want_s["out"])
        else:
            assert_outputs_match(got_s["out"], want_s["out"], TOL)


def test_selection_against_cpu_oracle():
    from oracle import risa_oracle as O
    from risaattention_b200.sparse import select_retained_mass_csr

    g = torch.Generator(device="cuda").manual_seed(3)
    masses = torch.rand(37, 70, device="cuda", generator=g) ** 4
    masses[5, 10:] = 0
    for theta in (0.3, 0.99, 1.0):
        ro, bi, mm = select_retained_mass_csr(masses, theta)
        oro, obi, omm = O.select_retained_mass(masses.cpu(), theta)
        assert torch.equal(ro.cpu(), oro) and torch.equal(bi.cpu(), obi)
        assert abs(mm - omm) < 1e-12


@pytest.mark.parametrize("dtype", [torch.bool, torch.float16, torch.bfloat16, torch.float32])
def test_key_mask_tiles(ref, dtype):
    from risaattention_b200 import _backend

    lk = 1153
    storage = torch.zeros(2, 4, 1, 2 * lk, device="cuda", dtype=dtype)
    mask = storage[..., ::2]
    visible = torch.ones(2, 4, 1, lk, device="cuda", dtype=torch.bool)
    visible[..., :128] = False
    visible[..., 384:768] = False
    visible[0, 1] = False
    visible[1, 2, :, -1] = False
    visible[..., 897:913] = False
    if dtype == torch.bool:
        mask.copy_(visible)
    else:
        mask.copy_(torch.linspace(-1, 2, lk, device="cuda"))
        mask.masked_fill_(~visible, -torch.inf)
    mask = mask.expand(2, 4, 300, lk)
    for tile in (64, 128):
        tiles = torch.empty(2, 4, -(-lk // tile) + 1, dtype=torch.int32, device="cuda")
        _backend._C.prepare_key_mask_tiles(mask, tiles, tile,
                                           torch.cuda.current_stream().cuda_stream)
        want = ref.key_mask_tiles(mask, tile)
        # defined content: the count in the last slot and that many ascending tile ids in front
        # (what lies between is scratch in both implementations)
        assert torch.equal(tiles[..., -1], want[..., -1])
        listed = torch.arange(tiles.shape[-1] - 1, device="cuda") < want[..., -1:]
        assert torch.equal(tiles[..., :-1][listed], want[..., :-1][listed])
        assert int(want[0, 1, -1]) == 0  # a fully hidden head lists nothing


def test_key_mask_tile_list_attention(ref):
    d, lq, lk, hq, hkv, cta_k = 128, 300, 1153, 4, 2, 128
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, b=2, seed=9)
    visible = torch.ones(2, hq, 1, lk, device="cuda", dtype=torch.bool)
    visible[..., :128] = False
    visible[..., 384:768] = False
    visible[0, 1] = False
    visible[..., 897:913] = False
    mask = visible.expand(2, hq, lq, lk)
    tiles = ref.key_mask_tiles(mask, cta_k)
    want = ref.attention(pk, sm_scale=d ** -0.5, mask=mask, want_lse=True, key_mask_tiles=tiles)
    got = _ours(pk, sm_scale=d ** -0.5, path=1, mask=mask, want_lse=True, tiles=tiles)
    assert_outputs_match(got["out"], want["out"], TOL)
    assert torch.count_nonzero(got["out"][0, 1]) == 0
    assert torch.isneginf(got["lse"][0, 1]).all()


def test_attention_against_cpu_oracle(ref):
    """The CPU restatement reproduces the GPU path within its budget (exp2 / reciprocal are
    approximate on the GPU): outputs within 2e-3 x RMS, LSE within 1e-3."""
    from oracle import risa_oracle as O

    d, lq, lk, hq, hkv, cta_k = 128, 200, 1153, 2, 1, 128
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, seed=21)
    got = _ours(pk, sm_scale=d ** -0.5, path=1, want_lse=True, capture=True)
    cpu = {k_: (v_.cpu() if torch.is_tensor(v_) else v_) for k_, v_ in pk.items()}
    want = O.attention(cpu["q"], cpu["k"], cpu["v"], cpu["q_scale"], cpu["k_scale"],
                       cpu["v_scale"], cpu["v_center"], cta_k=cta_k, sm_scale=d ** -0.5,
                       want_lse=True, capture=True)
    assert rel_max_err(got["out"].cpu(), want["out"]) <= TOL
    torch.testing.assert_close(got["lse"].cpu(), want["lse"], rtol=0, atol=1e-3)
    n = hq * 2 * 10
    torch.testing.assert_close(got["workspace"][:n].cpu(), want["workspace"][:n], rtol=1e-4,
                               atol=1e-4)
