"""Tensor-core attention kernel (tcgen05 + TMA) against the row-per-thread kernel and the
reference's own kernels: probabilities are exact integers on both paths, so capture statistics,
block masses and tile sets must be bit-identical; dense outputs agree within the output tolerance
(the dense path keeps one denominator partial instead of four)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.test_gpu_attention import TOL, _ours, _packed  # noqa: E402
from tests.util import assert_outputs_match  # noqa: E402


def _status():
    from risaattention_b200 import _backend

    _backend._C.device_status()


SHAPES = [
    # lq, lk, hq, hkv, batch
    (128, 1152, 1, 1, 1),
    (300, 1153, 4, 2, 1),
    (137, 2049, 2, 1, 2),
    (1000, 4096, 4, 4, 1),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_tc_dense_matches_rows_and_reference(ref, shape, causal):
    lq, lk, hq, hkv, b = shape
    _, _, _, pk = _packed(ref, 128, lq, lk, hq, hkv, 128, affine=True, seed=lq + lk, b=b)
    for scale in (128 ** -0.5, -0.125):
        want = ref.attention(pk, sm_scale=scale, is_causal=causal, want_lse=True)
        rows = _ours(pk, sm_scale=scale, path=1, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=scale, path=0, is_causal=causal, want_lse=True)
        _status()
        assert_outputs_match(got["out"], want["out"], TOL)
        assert_outputs_match(got["out"], rows["out"], TOL)
        torch.testing.assert_close(got["lse"], want["lse"], rtol=0, atol=2e-4)


@pytest.mark.parametrize("shape", SHAPES[:3])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_capture_bit_exact(ref, shape, causal):
    from risaattention_b200.sparse import select_retained_mass_csr

    lq, lk, hq, hkv, b = shape
    _, _, _, pk = _packed(ref, 128, lq, lk, hq, hkv, 128, seed=3 + lq, b=b)
    scale = 128 ** -0.5
    want = ref.attention(pk, sm_scale=scale, is_causal=causal, capture=True)
    got = _ours(pk, sm_scale=scale, path=0, is_causal=causal, capture=True)
    _status()
    assert torch.equal(got["workspace"].view(torch.int32), want["workspace"].view(torch.int32))
    assert torch.equal(got["out"], want["out"])
    n_q, n_k = -(-lq // 128), -(-lk // 128)
    masses = got["workspace"][: b * hq * n_q * n_k].view(-1, n_k)
    ro, bi, _ = select_retained_mass_csr(masses, 0.9)
    rro, rbi, _ = ref.select_retained_mass(want["workspace"][: b * hq * n_q * n_k].view(-1, n_k),
                                           0.9)
    assert torch.equal(ro, rro) and torch.equal(bi, rbi)
    want_s = ref.attention(pk, sm_scale=scale, is_causal=causal, row_offsets=rro,
                           block_indices=rbi)
    got_s = _ours(pk, sm_scale=scale, path=0, is_causal=causal, row_offsets=ro, block_indices=bi)
    _status()
    assert_outputs_match(got_s["out"], want_s["out"], TOL)


def test_tc_fp16_output_and_nhd_layout(ref):
    from risaattention_b200 import _backend

    _, _, _, pk = _packed(ref, 128, 300, 1300, 4, 2, 128, seed=77)
    want = ref.attention(pk, sm_scale=0.1, out_dtype=torch.float16)
    got = _ours(pk, sm_scale=0.1, path=0, out_dtype=torch.float16)
    _status()
    assert_outputs_match(got["out"], want["out"], TOL)
    out = torch.empty(1, 300, 4, 128, dtype=torch.bfloat16, device="cuda").permute(0, 2, 1, 3)
    _backend._C.risa_sdpa_prequantized(
        pk["q"], pk["k"], pk["v"], out, pk["q_scale"], pk["k_scale"], pk["v_scale"],
        pk["v_center"], 128, 0.1, 2, torch.cuda.current_stream().cuda_stream)
    _status()
    assert_outputs_match(out, ref.attention(pk, sm_scale=0.1)["out"], TOL)


MASK_SHAPES = [
    # lq, lk, hq, hkv, cta_k
    (137, 263, 2, 1, 64),
    (300, 1153, 4, 2, 128),
    (260, 1000, 4, 4, 64),
    (128, 129, 1, 1, 64),
]


@pytest.mark.parametrize("shape", MASK_SHAPES)
@pytest.mark.parametrize("mask_kind", ["none", "key_bias", "row_bool", "bias_4d"])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_masks_and_64_key_tiles(ref, shape, mask_kind, causal):
    """Every mask form and both key-tile widths on the tensor-core path, against the reference's
    kernels and the row kernel: outputs within 2e-3 x RMS, -inf rows identical, LSE within 2e-4
    (5e-4 with a mask: masked scores may differ from the reference's in the last FP32 bit, which
    can flip single U8 probability codes, and this path keeps one denominator partial)."""
    from tests.test_gpu_attention import _masks

    lq, lk, hq, hkv, cta_k = shape
    if mask_kind in ("row_bool", "bias_4d") and cta_k == 128:
        pytest.skip("per-query masks always use 64-key tiles")
    _, _, _, pk = _packed(ref, 128, lq, lk, hq, hkv, cta_k, affine=True, seed=lq + lk)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    for scale in (128 ** -0.5, 0.0, -0.125):
        want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, want_lse=True)
        rows = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, want_lse=True)
        _status()
        assert_outputs_match(got["out"], want["out"], TOL)
        assert_outputs_match(got["out"], rows["out"], TOL)
        assert torch.equal(torch.isneginf(got["lse"]), torch.isneginf(want["lse"]))
        fin = torch.isfinite(want["lse"])
        torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0,
                                   atol=2e-4 if mask_kind == "none" else 5e-4)
        if mask_kind == "row_bool":
            assert torch.count_nonzero(got["out"][:, :, 0]) == 0


@pytest.mark.parametrize("shape", MASK_SHAPES[:3])
@pytest.mark.parametrize("mask_kind", ["none", "key_bias"])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_capture_64_key_tiles_and_masks(ref, shape, mask_kind, causal):
    """Capture on the tensor-core path: the whole workspace bit for bit without a mask and against
    the row kernel with one (same arithmetic); against the reference masked masses agree to 1e-4
    (its compiler fuses score * scale + bias differently per instantiation)."""
    from risaattention_b200.sparse import select_retained_mass_csr
    from tests.test_gpu_attention import _masks

    lq, lk, hq, hkv, cta_k = shape
    _, _, _, pk = _packed(ref, 128, lq, lk, hq, hkv, cta_k, seed=5 + lk)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    scale = 128 ** -0.5
    want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, capture=True)
    rows = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, capture=True)
    got = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, capture=True)
    _status()
    assert torch.equal(got["workspace"].view(torch.int32), rows["workspace"].view(torch.int32))
    assert torch.equal(got["out"], rows["out"])
    n_q, n_k = -(-lq // 128), -(-lk // cta_k)
    if mask_kind == "none":
        assert torch.equal(got["workspace"].view(torch.int32), want["workspace"].view(torch.int32))
    else:
        torch.testing.assert_close(got["workspace"][: hq * n_q * n_k],
                                   want["workspace"][: hq * n_q * n_k], rtol=1e-4, atol=1e-5)
    masses = got["workspace"][: hq * n_q * n_k].view(-1, n_k)
    ro, bi, _ = select_retained_mass_csr(masses, 0.9)
    want_s = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, row_offsets=ro,
                           block_indices=bi)
    got_s = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, row_offsets=ro,
                  block_indices=bi)
    _status()
    assert_outputs_match(got_s["out"], want_s["out"], TOL)


@pytest.mark.parametrize("cta_k", [64, 128])
def test_tc_key_mask_tile_list(ref, cta_k):
    d, lq, lk, hq, hkv = 128, 300, 1153, 4, 2
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, b=2, seed=9)
    visible = torch.ones(2, hq, 1, lk, device="cuda", dtype=torch.bool)
    visible[..., :128] = False
    visible[..., 384:768] = False
    visible[0, 1] = False
    visible[..., 897:913] = False
    visible[1, 3, :, 1000:] = False  # the list ends before the last key tile
    mask = visible.expand(2, hq, lq, lk)
    tiles = ref.key_mask_tiles(mask, cta_k)
    want = ref.attention(pk, sm_scale=d ** -0.5, mask=mask, want_lse=True, key_mask_tiles=tiles)
    got = _ours(pk, sm_scale=d ** -0.5, path=0, mask=mask, want_lse=True, tiles=tiles)
    _status()
    assert_outputs_match(got["out"], want["out"], TOL)
    assert torch.count_nonzero(got["out"][0, 1]) == 0
    assert torch.isneginf(got["lse"][0, 1]).all()
    fin = torch.isfinite(want["lse"])
    torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0, atol=5e-4)


D64_SHAPES = [
    # lq, lk, hq, hkv
    (137, 263, 2, 1),
    (300, 1153, 4, 2),
    (128, 2048, 2, 2),
]


@pytest.mark.parametrize("shape", D64_SHAPES)
@pytest.mark.parametrize("mask_kind", ["none", "key_bias", "bias_4d"])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_head_dim_64(ref, shape, mask_kind, causal):
    """head_dim 64 (64-byte operand rows, 64-byte swizzle) on the tensor-core path."""
    from tests.test_gpu_attention import _masks

    lq, lk, hq, hkv = shape
    _, _, _, pk = _packed(ref, 64, lq, lk, hq, hkv, 64, affine=True, seed=lq + lk)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    for scale in (64 ** -0.5, -0.125):
        want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, want_lse=True)
        rows = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, want_lse=True)
        _status()
        assert_outputs_match(got["out"], want["out"], TOL)
        assert_outputs_match(got["out"], rows["out"], TOL)
        fin = torch.isfinite(want["lse"])
        torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0,
                                   atol=2e-4 if mask_kind == "none" else 5e-4)


@pytest.mark.parametrize("causal", [False, True])
def test_tc_head_dim_64_capture_bit_exact(ref, causal):
    from risaattention_b200.sparse import select_retained_mass_csr

    lq, lk, hq, hkv = 300, 1153, 4, 2
    _, _, _, pk = _packed(ref, 64, lq, lk, hq, hkv, 64, seed=21)
    want = ref.attention(pk, sm_scale=0.125, is_causal=causal, capture=True)
    got = _ours(pk, sm_scale=0.125, path=0, is_causal=causal, capture=True)
    _status()
    assert torch.equal(got["workspace"].view(torch.int32), want["workspace"].view(torch.int32))
    assert torch.equal(got["out"], want["out"])
    n_q, n_k = -(-lq // 128), -(-lk // 64)
    masses = got["workspace"][: hq * n_q * n_k].view(-1, n_k)
    ro, bi, _ = select_retained_mass_csr(masses, 0.9)
    want_s = ref.attention(pk, sm_scale=0.125, is_causal=causal, row_offsets=ro, block_indices=bi)
    got_s = _ours(pk, sm_scale=0.125, path=0, is_causal=causal, row_offsets=ro, block_indices=bi)
    _status()
    assert_outputs_match(got_s["out"], want_s["out"], TOL)


@pytest.mark.parametrize("cta_k", [64, 128])
@pytest.mark.parametrize("mask_kind", ["none", "key_bias", "bias_4d"])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_head_dim_256(ref, cta_k, mask_kind, causal):
    """head_dim 256: two CTAs per (query block, head), each contracting over all 256 channels
    (two column panels) and producing 128 output channels."""
    from tests.test_gpu_attention import _masks

    if mask_kind == "bias_4d" and cta_k == 128:
        pytest.skip("per-query masks always use 64-key tiles")
    lq, lk, hq, hkv = 300, 1153, 4, 2
    _, _, _, pk = _packed(ref, 256, lq, lk, hq, hkv, cta_k, affine=True, seed=cta_k)
    mask = _masks(mask_kind, 1, hq, lq, lk)
    for scale in (256 ** -0.5, -0.125):
        want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, want_lse=True)
        rows = _ours(pk, sm_scale=scale, path=1, mask=mask, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, want_lse=True)
        _status()
        assert_outputs_match(got["out"], want["out"], TOL)
        assert_outputs_match(got["out"], rows["out"], TOL)
        fin = torch.isfinite(want["lse"])
        torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0,
                                   atol=2e-4 if mask_kind == "none" else 5e-4)


@pytest.mark.parametrize("cta_k", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_tc_head_dim_256_capture_bit_exact(ref, cta_k, causal):
    lq, lk, hq, hkv = 300, 1153, 4, 2
    _, _, _, pk = _packed(ref, 256, lq, lk, hq, hkv, cta_k, seed=31)
    want = ref.attention(pk, sm_scale=0.0625, is_causal=causal, capture=True)
    got = _ours(pk, sm_scale=0.0625, path=0, is_causal=causal, capture=True)
    _status()
    assert torch.equal(got["workspace"].view(torch.int32), want["workspace"].view(torch.int32))
    assert torch.equal(got["out"], want["out"])


SELECT_SHAPES = [
    # d, lq, lk, hq, hkv, batch, cta_k
    (128, 300, 1153, 4, 2, 1, 128),
    (128, 137, 2049, 2, 1, 2, 128),
    (128, 260, 1000, 4, 4, 1, 64),
    (64, 200, 700, 2, 1, 1, 64),
    (256, 130, 1100, 2, 2, 1, 128),
    (256, 137, 263, 2, 1, 1, 64),
    (128, 1000, 4096, 4, 4, 1, 128),
]


@pytest.mark.parametrize("shape", SELECT_SHAPES)
@pytest.mark.parametrize("variant", ["plain", "causal", "key_bias"])
def test_in_pass_selection_bit_exact(ref, shape, variant):
    """Pattern construction inside the attention launch: block masses, kept-tile sets, counts and
    the attention output itself are the reference's (capture workspace -> block-mass kernel ->
    torch.sort -> selector) bit for bit, for several thresholds including theta = 1."""
    from risaattention_b200 import _backend
    from tests.test_gpu_attention import _masks

    d, lq, lk, hq, hkv, b, cta_k = shape
    _, _, _, pk = _packed(ref, d, lq, lk, hq, hkv, cta_k, seed=11 + lk, b=b)
    causal = variant == "causal"
    mask = _masks("key_bias", b, hq, lq, lk) if variant == "key_bias" else None
    scale = d ** -0.5
    want = ref.attention(pk, sm_scale=scale, mask=mask, is_causal=causal, capture=True)
    n_q, n_k = -(-lq // 128), -(-lk // cta_k)
    rows, words = b * hq * n_q, -(-n_k // 32)
    want_masses = want["workspace"][: rows * n_k].view(rows, n_k)
    C = _backend._C
    assert n_k <= C.select_max_key_tiles(cta_k)
    stream = torch.cuda.current_stream().cuda_stream
    for theta in (0.5, 0.9, 0.99, 1.0):
        out = torch.empty(b, hq, lq, d, dtype=torch.bfloat16, device="cuda")
        counts = torch.empty(rows, dtype=torch.int32, device="cuda")
        bitmaps = torch.empty(rows, words, dtype=torch.int32, device="cuda")
        totals = torch.empty(rows, 2, dtype=torch.float64, device="cuda")
        masses = torch.empty(rows, n_k, device="cuda")
        scratch = torch.empty(C.select_scratch_size(lk, cta_k), dtype=torch.uint8, device="cuda")
        C.risa_sdpa_select(pk["q"], pk["k"], pk["v"], out, pk["q_scale"], pk["k_scale"],
                           pk["v_scale"], pk["v_center"], cta_k, scale, 2, stream, theta, scratch,
                           counts, bitmaps, totals, attn_mask=mask, is_causal=causal,
                           block_masses=masses)
        offsets = torch.empty(rows + 1, dtype=torch.int32, device="cuda")
        storage = torch.empty(rows * n_k, dtype=torch.int32, device="cuda")
        summary = torch.empty(3, dtype=torch.float64, device="cuda")
        C.pack_selected(counts, bitmaps, totals, offsets, storage, summary, n_k, stream)
        torch.cuda.synchronize()
        _status()
        if variant == "key_bias":
            # masked scores may differ from the reference's in the last FP32 bit (its compiler
            # fuses score * scale + bias per instantiation): masses to 1e-4, selection against
            # this library's own capture path instead
            torch.testing.assert_close(masses, want_masses, rtol=0, atol=1e-4)
            own = _ours(pk, sm_scale=scale, path=0, mask=mask, is_causal=causal, capture=True)
            base = own["workspace"][: rows * n_k].view(rows, n_k)
            assert torch.equal(masses, base)
            assert torch.equal(out, own["out"])
        else:
            base = want_masses
            assert torch.equal(masses, want_masses)
            assert torch.equal(out, want["out"])
        rro, rbi, rmeasured = ref.select_retained_mass(base, theta)
        kept = int(summary[2])
        assert torch.equal(offsets, rro) and torch.equal(storage[:kept], rbi)
        assert abs(float(summary[0]) / max(float(summary[1]), 1e-20) - rmeasured) < 1e-12
        assert torch.equal(counts, rro[1:] - rro[:-1])


def test_in_pass_selection_orders_equal_masses_by_tile_id(ref):
    """Equal block masses (constant keys: every tile of a row weighs the same) are kept in
    ascending tile order, so the kept set is the first `count` tiles; the count itself is the
    reference selector's."""
    import risaattention_b200 as risa

    q = torch.randn(1, 2, 256, 128, device="cuda").bfloat16()
    k = torch.ones(1, 1, 2048, 128, device="cuda").bfloat16()
    v = torch.randn(1, 1, 2048, 128, device="cuda").bfloat16()
    _, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.5)
    counts = (pattern.row_offsets[1:] - pattern.row_offsets[:-1]).tolist()
    assert counts == [8] * 4
    assert pattern.block_indices.view(4, 8).tolist() == [list(range(8))] * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.bool])
@pytest.mark.parametrize("offset", [0, 3])
def test_per_query_mask_staging_forms(ref, dtype, offset):
    """Per-query masks of every element type, with rows that start on 16-byte boundaries (vector
    staging) and rows that do not (element-wise staging), against the reference's kernels."""
    from tests.test_gpu_attention import _packed

    lq, lk, hq, hkv = 256, 1024, 4, 2
    _, _, _, pk = _packed(ref, 128, lq, lk, hq, hkv, 64, affine=True, seed=91)
    g = torch.Generator(device="cuda").manual_seed(92)
    storage = torch.empty(1, hq, lq, lk + 16, device="cuda", dtype=dtype)
    mask = storage[..., offset:offset + lk]
    if dtype == torch.bool:
        mask.copy_(torch.rand(1, hq, lq, lk, device="cuda", generator=g) > 0.3)
        mask[:, :, 5] = False
    else:
        mask.copy_(torch.randn(1, hq, lq, lk, device="cuda", generator=g))
        mask[:, :, :, 7::11] = float("-inf")
    for causal in (False, True):
        want = ref.attention(pk, sm_scale=128 ** -0.5, mask=mask, is_causal=causal, want_lse=True)
        got = _ours(pk, sm_scale=128 ** -0.5, path=0, mask=mask, is_causal=causal, want_lse=True)
        _status()
        assert_outputs_match(got["out"], want["out"], TOL)
        assert torch.equal(torch.isneginf(got["lse"]), torch.isneginf(want["lse"]))
        fin = torch.isfinite(want["lse"])
        torch.testing.assert_close(got["lse"][fin], want["lse"][fin], rtol=0, atol=5e-4)


@pytest.mark.parametrize("shape", [
    # dim, q heads, kv heads, length: CTA counts that leave a small last wave on a 148-SM GPU
    (128, 16, 4, 4096),   # 512 CTAs: 68 in the last wave, two key-range parts each
    (128, 5, 5, 4096),    # 160 CTAs: 12 in the last wave, four parts each
    (256, 5, 1, 4096),    # two CTAs per (query block, head): 320 CTAs, 24 in the last wave
    (64, 5, 5, 4096),     # 64-key tiles, 64 output channels
    (128, 16, 4, 4000),   # ragged: the last query block and the last key tile are partial
])
def test_split_last_wave_matches_whole_ctas(ref, shape):
    """The Python routes cut the CTAs of a small last wave into key-range parts and merge them;
    risa_b200_attention (no scratch) runs whole CTAs.  Same packed operands: every element within
    the output tolerance, almost all bit-identical (only rows of split CTAs can differ, by the last
    place of their FP32 sums), and everything within tolerance of the reference's kernel."""
    import ctypes

    import risaattention_b200 as risa
    from oracle import ref_gpu
    from risaattention_b200 import _backend

    dim, hq, hkv, length = shape
    g = torch.Generator(device="cuda").manual_seed(length + dim + hq)
    q = torch.randn(1, hq, length, dim, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, hkv, length, dim, device="cuda", generator=g).bfloat16()
    v = torch.randn(1, hkv, length, dim, device="cuda", generator=g).bfloat16()
    one_call = risa.int8_attention(q, k, v)
    packed = risa.prequantize_int8_attention(q, k, v)
    two_calls = risa.int8_attention_from_prequantized(packed)
    C = _backend._ABI
    assert C.lib.risa_b200_attention_scratch_size(1, hq, length, length, dim, packed.cta_k) > 0, \
        "shape was meant to leave a small last wave"
    whole = torch.empty_like(one_call)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    C._check(C.lib.risa_b200_attention(
        p(packed.q), p(packed.k), p(packed.v), p(whole), p(packed.q_scale), p(packed.k_scale),
        p(packed.v_scale), p(packed.v_center), None, 0, 0, 0, 0, -1, packed.cta_k, 1, length,
        length, hq, hkv, dim, whole.stride(0), whole.stride(2), whole.stride(1),
        packed.attention_scale, 2, None, None, None, 0, None, None,
        torch.cuda.current_stream().cuda_stream))
    # a scratch too small for the parts (sized for another GPU, say) must give whole CTAs
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    guarded = torch.empty_like(one_call)
    C._check(C.lib.risa_b200_attention_scratch(
        p(packed.q), p(packed.k), p(packed.v), p(guarded), p(packed.q_scale), p(packed.k_scale),
        p(packed.v_scale), p(packed.v_center), None, 0, 0, 0, 0, -1, packed.cta_k, 1, length,
        length, hq, hkv, dim, guarded.stride(0), guarded.stride(2), guarded.stride(1),
        packed.attention_scale, 2, None, None, None, 0, None, None, p(small), small.numel(),
        torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(guarded, whole)
    assert torch.equal(one_call, two_calls)  # same kernels, same split
    assert_outputs_match(one_call, whole, TOL)
    differing = (one_call != whole).float().mean()
    assert 0 < differing < 0.02, "the split rows should differ somewhere, and only there"
    want = torch.empty_like(whole)
    pk = ref_gpu.prequantize(q, k, v, cta_k=packed.cta_k)
    ref_gpu.attention(pk, sm_scale=dim ** -0.5, out=want)
    torch.cuda.synchronize()
    assert_outputs_match(one_call, want, TOL)
