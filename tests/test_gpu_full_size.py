"""Parity at the benchmark specification's stated sizes, against the reference's own kernels
(oracle/_ref) on the same seeded inputs:

* the dense sweep, Lq = Lk in {512 ... 32768} x {absmax, midpoint_affine} x seeds 0, 1, 2, all 16
  query heads: codes, scales and anchors bit for bit, outputs within 2e-3 x RMS (+ 1 ulp of bf16);
* one 32K pattern construction per sparse workload: the whole 1.08 GB capture workspace (64-bit
  offsets) and the CSR tile sets at theta = 0.99 bit for bit, plus sparse reuse on drifted inputs;
* the video-DiT shape at L = 32760 (ragged last tile after 255 full ones) with one GPU's 5 heads;
* the edge sweep at Hq 32, Hkv 8, Lq 4096, Lk 16384 for head_dim 64 and 256: causal, additive
  [B,Hq,Lq,Lk] bias, boolean mask with fully masked rows, batch 2 with LSE.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import synthetic  # noqa: E402
from tests.util import assert_outputs_match  # noqa: E402

TOL = 2e-3  # max |ours - reference| / RMS(reference output), plus one ulp of the 16-bit output


def _status():
    from risaattention_b200 import _backend

    _backend._C.device_status()


def _codes_equal(pk, want, centres_exact=True):
    for name, ours in (("q", pk.q), ("k", pk.k), ("v", pk.v), ("q_scale", pk.q_scale),
                       ("k_scale", pk.k_scale), ("v_scale", pk.v_scale)):
        assert torch.equal(ours.reshape(-1), want[name].reshape(-1)), name
    if centres_exact:
        assert torch.equal(pk.v_center, want["v_center"])
    else:
        # midpoint-affine centre = midpoint + scale * mean residual, one FMA.  Identical to the
        # reference's in more than 99 % of the channels; elsewhere the two terms are one unit in
        # the last place of the larger one apart (the terms cancel when the midpoint is near zero,
        # so the bound is taken at |centre| + scale, not at the centre itself).
        ref_c = want["v_center"]
        size = ref_c.abs() + want["v_scale"]
        ulp = torch.nextafter(size, torch.full_like(size, 9e9)) - size
        assert ((pk.v_center - ref_c).abs() <= ulp).all()
        assert (pk.v_center != ref_c).float().mean() < 0.01


@pytest.mark.parametrize("seed", [0, 1, 2])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
@pytest.mark.parametrize("length", [512, 1024, 2048, 4096, 8192, 16384, 32768])
def test_dense_sweep(ref, length, mode, seed):
    q, k, v = synthetic.dense_inputs(length, "cuda", seed=seed)
    affine = mode == "midpoint_affine"
    cta_k = 128 if length > 1024 else 64
    want_pk = ref.prequantize(q, k, v, cta_k=cta_k, midpoint_affine=affine)
    pk = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
    assert pk.cta_k == cta_k
    _codes_equal(pk, want_pk, centres_exact=not affine)
    want = ref.attention(want_pk, sm_scale=128 ** -0.5)
    got = risa.int8_attention(q, k, v, v_quantization=mode)
    _status()
    assert_outputs_match(got, want["out"], TOL)
    assert_outputs_match(risa.int8_attention_from_prequantized(pk), want["out"], TOL)


@pytest.mark.parametrize("workload", ["video_blocks", "block_centroids"])
def test_pattern_construction_32k(ref, workload):
    """Capture statistics, block masses and tile sets of a full 32K call are the reference's bit
    for bit; the retained support is reused on drifted inputs and matches the reference's sparse
    kernel run on the same tile lists."""
    length, heads = 32768, 16
    make = synthetic.video_block_inputs if workload == "video_blocks" \
        else synthetic.block_centroid_inputs
    q, k, v, g = make(length, "cuda")
    want_pk = ref.prequantize(q, k, v, cta_k=128)
    pk = risa.prequantize_int8_attention(q, k, v)
    _codes_equal(pk, want_pk)
    out, pattern = risa.construct_sparse_int8_attention_from_prequantized(pk, theta=0.99)
    _status()
    cap = ref.attention(want_pk, sm_scale=128 ** -0.5, capture=True)
    n = length // 128
    masses = cap["workspace"][: heads * n * n].view(-1, n)
    rro, rbi, rmeasured = ref.select_retained_mass(masses, 0.99)
    assert torch.equal(pattern.row_offsets, rro)
    assert torch.equal(pattern.block_indices, rbi)
    assert abs(pattern.measured_retained_mass - rmeasured) < 1e-12
    assert torch.equal(out, cap["out"])  # the capture pass keeps the reference's FP32 order
    del cap, masses

    # the raw workspace: block masses, per-tile (numerator, maximum) pairs, final (m, d) per row
    from tests.test_gpu_attention import _ours
    got = _ours(want_pk, sm_scale=128 ** -0.5, path=0, capture=True)
    _status()
    cap = ref.attention(want_pk, sm_scale=128 ** -0.5, capture=True)
    assert got["workspace"].numel() == heads * n * n + heads * length * (2 * n + 2) > 2 ** 28
    assert torch.equal(got["workspace"].view(torch.int32), cap["workspace"].view(torch.int32))
    rows = got["workspace"][: heads * n * n].view(-1, n).sum(-1)
    torch.testing.assert_close(rows, torch.full_like(rows, 128.0), rtol=0, atol=2e-3)
    del cap, got

    kind = "additive" if workload == "video_blocks" else "blend"
    q2, k2, v2 = (synthetic.drift(t, g, kind) for t in (q, k, v))
    reuse = risa.sparse_int8_attention(q2, k2, v2, pattern)
    _status()
    pk2 = ref.prequantize(q2, k2, v2, cta_k=128)
    if pattern.sparsity < 0.05:
        want = ref.attention(pk2, sm_scale=128 ** -0.5)
    else:
        want = ref.attention(pk2, sm_scale=128 ** -0.5, row_offsets=rro, block_indices=rbi)
    assert_outputs_match(reuse, want["out"], TOL)


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_video_dit_full_length(ref, mode):
    """One GPU's share of the video-DiT configuration: 5 of the 40 heads at L = 32760."""
    heads, length = 5, 32760
    q, k, v = synthetic.video_dit_inputs(heads, "cuda", seq_len=length)
    affine = mode == "midpoint_affine"
    want_pk = ref.prequantize(q, k, v, cta_k=128, midpoint_affine=affine)
    pk = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
    _codes_equal(pk, want_pk, centres_exact=not affine)
    want = ref.attention(want_pk, sm_scale=128 ** -0.5)
    got = risa.int8_attention(q, k, v, v_quantization=mode)
    _status()
    assert_outputs_match(got, want["out"], TOL)

    out, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.99, v_quantization=mode)
    _status()
    cap = ref.attention(want_pk, sm_scale=128 ** -0.5, capture=True)
    n = 256
    rro, rbi, _ = ref.select_retained_mass(cap["workspace"][: heads * n * n].view(-1, n), 0.99)
    assert torch.equal(pattern.row_offsets, rro) and torch.equal(pattern.block_indices, rbi)
    assert torch.equal(out, cap["out"])
    del cap
    from tests.test_gpu_attention import _ours
    got_s = _ours(want_pk, sm_scale=128 ** -0.5, path=0, row_offsets=rro, block_indices=rbi)
    _status()
    want_s = ref.attention(want_pk, sm_scale=128 ** -0.5, row_offsets=rro, block_indices=rbi)
    assert_outputs_match(got_s["out"], want_s["out"], TOL)


@pytest.mark.parametrize("dim", [64, 256])
@pytest.mark.parametrize("feature", ["causal", "bias", "bool_rows", "batch2_lse"])
def test_edge_sweep_full_size(ref, dim, feature):
    hq, hkv, lq, lk = 32, 8, 4096, 16384
    b = 2 if feature in ("bool_rows", "batch2_lse") else 1
    q, k, v = synthetic.dense_inputs(lq, "cuda", seed=dim, q_heads=hq, kv_heads=hkv,
                                     head_dim=dim, batch=b, kv_len=lk)
    g = torch.Generator(device="cuda").manual_seed(dim + 1)
    mask, causal, dead = None, feature == "causal", None
    if feature == "bias":
        mask = torch.randn(b, hq, lq, lk, device="cuda", generator=g)
    elif feature == "bool_rows":
        mask = torch.ones(b, hq, lq, lk, device="cuda", dtype=torch.bool)
        dead = torch.randperm(lq, device="cuda", generator=g)[: lq // 10]
        mask[:, :, dead] = False
    pk = risa.prequantize_int8_attention(q, k, v, attn_mask=mask, is_causal=causal,
                                         return_lse=True)
    out, lse = risa.int8_attention_from_prequantized(pk, return_lse=True)
    _status()
    cta_k = pk.cta_k
    assert cta_k == (64 if (mask is not None or dim == 64) else 128)
    want_pk = ref.prequantize(q, k, v, cta_k=cta_k)
    _codes_equal(pk, want_pk)
    want = ref.attention(want_pk, sm_scale=dim ** -0.5, mask=mask, is_causal=causal,
                         want_lse=True)
    assert_outputs_match(out, want["out"], TOL)
    want_lse = want["lse"] + ref.lse_shift(q, k, want_pk["anchors"], dim ** -0.5)
    assert torch.equal(torch.isneginf(lse), torch.isneginf(want_lse))
    fin = torch.isfinite(want_lse)
    torch.testing.assert_close(lse[fin], want_lse[fin], rtol=0, atol=5e-4)
    if dead is not None:
        assert torch.count_nonzero(out[:, :, dead]) == 0
        assert torch.isneginf(lse[:, :, dead]).all()
    if feature == "batch2_lse":
        direct, lse_direct = risa.int8_attention(q, k, v, return_lse=True)
        assert torch.equal(out, direct) and torch.equal(lse, lse_direct)


@pytest.fixture(scope="module")
def wide_operands():
    """Packed operands whose query-head stride is 2^30 + 8192 bytes, so the last of the five heads
    starts beyond 4 GiB in Q and beyond 8 GiB in the FP16 output (the reference keeps the same
    case as an opt-in test: tests/cuda/test_large_offsets.py:22-37)."""
    if torch.cuda.mem_get_info()[0] < 24 * 1024 ** 3:
        pytest.skip("needs 24 GiB of free device memory")
    length, heads, dim = (1 << 30) // 64 + 128, 5, 64
    q = torch.zeros((1, heads, length, dim), dtype=torch.int8, device="cuda")
    q_scale = torch.ones((1, heads, -(-length // 128) * 32), device="cuda")
    assert (heads - 1) * q.stride(1) > (1 << 32) - 1
    yield q, q_scale
    del q, q_scale
    torch.cuda.empty_cache()


@pytest.mark.parametrize("keys", [1, 128])
@pytest.mark.parametrize("route", ["dense", "sparse", "capture"])
def test_head_offsets_beyond_four_gibibytes(wide_operands, route, keys):
    """Every output element of a 5 x 16.8M-query call is checked: with zero scores and the value
    100 x 0.2 under every key, each row is exactly 20.  One key runs the row-per-thread kernel (the
    packed V row is shorter than a 128-key slab), 128 keys the tensor-core kernel with two tiles;
    the sparse route keeps the first tile of every row, the capture route also checks the block
    masses (128 queries per block, spread evenly over the key tiles)."""
    from risaattention_b200 import _backend

    q, q_scale = wide_operands
    heads, length, dim = q.shape[1], q.shape[2], q.shape[3]
    tiles = -(-keys // 64)
    k = torch.zeros((1, 1, keys, dim), dtype=torch.int8, device="cuda")
    v = torch.zeros((dim, tiles * 64), dtype=torch.int8, device="cuda")
    v[:, :keys] = 100
    k_scale = torch.ones((1, 1, tiles * 4), device="cuda")
    v_scale = torch.full((dim,), 0.2, device="cuda")
    v_center = torch.zeros_like(v_scale)
    output = torch.empty(q.shape, dtype=torch.float16, device="cuda")
    rows = heads * -(-length // 128)
    extra = {}
    if route == "sparse":
        extra["sparse_row_offsets"] = torch.arange(rows + 1, device="cuda", dtype=torch.int32)
        extra["sparse_block_indices"] = torch.zeros(rows, device="cuda", dtype=torch.int32)
    elif route == "capture":
        workspace = torch.empty(rows * tiles + heads * length * (2 * tiles + 2), device="cuda")
        extra["block_mass"] = workspace
    _backend._C.risa_sdpa_prequantized(q, k, v, output, q_scale, k_scale, v_scale, v_center, 64,
                                       0.125, 1, torch.cuda.current_stream().cuda_stream, **extra)
    torch.cuda.synchronize()
    _status()
    assert output.amin().item() == 20.0
    assert output.amax().item() == 20.0
    if route == "capture":
        masses = workspace[: rows * tiles]
        torch.testing.assert_close(masses, torch.full_like(masses, 128.0 / tiles), rtol=0.0,
                                   atol=2e-5)
