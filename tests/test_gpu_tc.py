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
