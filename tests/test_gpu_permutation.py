"""K/V token permutations: quantising through the gather table (fuse_gather=True) must give the
packed operands of quantising a materialised gather (fuse_gather=False) bit for bit -- K codes and
scales, the sampled anchor, V codes, scales and residual-corrected centres -- for every input dtype,
head dim and memory layout, and the attention output must equal attention over the gathered K/V
(the reference pins the V part in tests/cuda/test_value_quantization.py:55-72)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import prepare_kv_permutation  # noqa: E402

FIELDS = ("q", "k", "v", "q_scale", "k_scale", "v_scale", "v_center")


def _tables(b, hkv, lk, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows = [torch.randperm(lk, device="cuda", generator=g) for _ in range(b * hkv)]
    return torch.stack(rows).view(b, hkv, lk)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("lk", [193, 1153, 2048])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_fused_gather_equals_materialised_gather(dtype, dim, lk, mode):
    b, hq, hkv, lq = 2, 4, 2, 137
    g = torch.Generator(device="cuda").manual_seed(lk + dim)
    q = torch.randn(b, hq, lq, dim, device="cuda", generator=g).to(dtype)
    # clustered keys so that the K anchor fires and its sampled rows go through the table too
    k = (torch.randn(b, hkv, lk, dim, device="cuda", generator=g) * 0.1 + 4).to(dtype)
    v = (torch.randn(b, hkv, lk, dim, device="cuda", generator=g) + 0.5).to(dtype)
    permutation = prepare_kv_permutation(_tables(b, hkv, lk, seed=lk))
    fused = risa.prequantize_int8_attention(q, k, v, kv_permutation=permutation,
                                            fuse_gather=True, v_quantization=mode)
    eager = risa.prequantize_int8_attention(q, k, v, kv_permutation=permutation,
                                            fuse_gather=False, v_quantization=mode)
    assert fused.kv_permuted and eager.kv_permuted
    for name in FIELDS:
        assert torch.equal(getattr(fused, name), getattr(eager, name)), name
    # the same packed operands as quantising the gathered tensors without any permutation
    rows = permutation.table().long()[..., None].expand_as(k)
    plain = risa.prequantize_int8_attention(q, k.gather(2, rows), v.gather(2, rows),
                                            v_quantization=mode)
    for name in FIELDS:
        assert torch.equal(getattr(fused, name), getattr(plain, name)), name
    out_fused = risa.int8_attention(q, k, v, kv_permutation=permutation, v_quantization=mode)
    out_plain = risa.int8_attention(q, k.gather(2, rows), v.gather(2, rows), v_quantization=mode)
    assert torch.equal(out_fused, out_plain)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", ["hnd", "nhd", "interleaved"])
def test_packed_values_match_materialised_permutation(dtype, layout):
    """Shapes and layouts of the reference's own permutation test."""
    q = torch.randn(1, 4, 17, 128, device="cuda", dtype=dtype)
    k, v = [torch.randn(1, 2, 2049, 128, device="cuda", dtype=dtype) for _ in range(2)]
    if layout == "nhd":
        v = v.transpose(1, 2).contiguous().transpose(1, 2)
    elif layout == "interleaved":
        storage = torch.empty(1, 2049, 3, 2, 128, device="cuda", dtype=dtype)
        v = storage[:, :, 1].transpose(1, 2).copy_(v)
    permutation = prepare_kv_permutation(_tables(1, 2, 2049, seed=3))
    fused = risa.prequantize_int8_attention(q, k, v, kv_permutation=permutation, fuse_gather=True)
    eager = risa.prequantize_int8_attention(q, k, v, kv_permutation=permutation, fuse_gather=False)
    for name in FIELDS:
        assert torch.equal(getattr(fused, name), getattr(eager, name)), name


def test_permutation_with_lse_and_contract():
    q = torch.randn(1, 4, 200, 128, device="cuda", dtype=torch.bfloat16)
    k, v = [torch.randn(1, 2, 1300, 128, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    table = _tables(1, 2, 1300, seed=9)
    permutation = prepare_kv_permutation(table)
    rows = table[..., None].expand_as(k)
    out, lse = risa.int8_attention(q, k, v, kv_permutation=permutation, return_lse=True)
    want, want_lse = risa.int8_attention(q, k.gather(2, rows), v.gather(2, rows), return_lse=True)
    assert torch.equal(out, want) and torch.equal(lse, want_lse)
    with pytest.raises(ValueError, match="exactly once"):
        prepare_kv_permutation(torch.zeros(1, 2, 1300, dtype=torch.int64, device="cuda"))
    with pytest.raises(ValueError, match="dense, unmasked, noncausal"):
        risa.int8_attention(q, k, v, kv_permutation=permutation, is_causal=True)
    with pytest.raises(TypeError, match="prepare_kv_permutation"):
        risa.int8_attention(q, k, v, kv_permutation=table)
    with pytest.raises(ValueError, match="must match K"):
        risa.int8_attention(q, k[:, :, :1200], v[:, :, :1200], kv_permutation=permutation)
    permutation.table()[0, 0, 0] = 5  # an in-place write after validation is detected
    with pytest.raises(ValueError, match="was modified"):
        risa.int8_attention(q, k, v, kv_permutation=permutation)
