"""The native object called the way the reference's Python runtime calls its ``_C`` module
(src/risa_attention/_execution.py:100-130,279-321, _quantization.py:120-157, sparse.py:23-48,
_key_mask.py:19-27): every tensor wrapped as a DLPack capsule, anchor scratch and gather table as
raw integer addresses, no V-quantiser workspace, key-mask tiles only as an optional keyword.  The
results must equal this package's own API on the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import _backend  # noqa: E402

CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


@pytest.fixture(params=["extension", "ctypes"])
def native(request):
    """Both host-side surfaces over the C-ABI: the PyTorch C++ extension (what the package uses)
    and the ctypes object."""
    return _backend._C if request.param == "extension" else _backend._ABI


def cap(t):
    """What the reference's wrap_for_dlpack produces for an ordinary CUDA tensor."""
    return None if t is None else torch.utils.dlpack.to_dlpack(t)


def _buffers(q, k, cta_k):
    b, hq, lq, d = q.shape
    hkv, lk = k.shape[1], k.shape[2]
    dev = q.device
    padded = -(-lk // cta_k) * cta_k
    return dict(
        q_int8=torch.empty(q.shape, dtype=torch.int8, device=dev),
        q_scale=torch.empty(b, hq, -(-lq // 128) * (64 if d == 256 else 32), device=dev),
        k_int8=torch.empty(k.shape, dtype=torch.int8, device=dev),
        k_scale=torch.empty(b, hkv, -(-lk // cta_k) * 4, device=dev),
        v_int8=torch.empty(b * hkv * d, padded, dtype=torch.int8, device=dev),
        v_scale=torch.empty(b * hkv * d, device=dev),
        v_center=torch.empty(b * hkv * d, device=dev),
        anchors=torch.empty(b, hkv, dtype=torch.int32, device=dev))


@pytest.mark.parametrize("lk", [700, 2304])
@pytest.mark.parametrize("causal", [False, True])
def test_risa_sdpa_called_like_the_reference(native, lk, causal):
    C = native
    g = torch.Generator(device="cuda").manual_seed(lk)
    q = torch.randn(2, 8, 300, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(2, 2, lk, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(2, 2, lk, 128, device="cuda", generator=g).bfloat16()
    cta_k = 128 if lk > 1024 else 64
    buf = _buffers(q, k, cta_k)
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    C.risa_sdpa(cap(q), cap(k), cap(v), cap(out), cap(buf["q_int8"]), cap(buf["q_scale"]),
                cap(buf["k_int8"]), cap(buf["k_scale"]), cap(buf["v_int8"]), cap(buf["v_scale"]),
                cap(buf["v_center"]), 128 ** -0.5, CODES[q.dtype], CODES[out.dtype], False,
                stream, buf["anchors"].data_ptr(), None, cta_k=cta_k, is_causal=causal)
    want = risa.int8_attention(q, k, v, is_causal=causal)
    assert torch.equal(out, want)
    # cta_k left at its default of 0 selects the same tile width (csrc/bindings.cpp:549-551)
    out2 = torch.empty_like(out)
    C.risa_sdpa(cap(q), cap(k), cap(v), cap(out2), cap(buf["q_int8"]), cap(buf["q_scale"]),
                cap(buf["k_int8"]), cap(buf["k_scale"]), cap(buf["v_int8"]), cap(buf["v_scale"]),
                cap(buf["v_center"]), 128 ** -0.5, CODES[q.dtype], CODES[out.dtype], False,
                stream, buf["anchors"].data_ptr(), is_causal=causal)
    assert torch.equal(out2, want)
    with pytest.raises(RuntimeError, match="anchor_indices scratch is required"):
        C.risa_sdpa(cap(q), cap(k), cap(v), cap(out2), cap(buf["q_int8"]), cap(buf["q_scale"]),
                    cap(buf["k_int8"]), cap(buf["k_scale"]), cap(buf["v_int8"]),
                    cap(buf["v_scale"]), cap(buf["v_center"]), 128 ** -0.5, 2, 2, False, stream, 0)


def test_masked_sdpa_with_key_mask_tiles_keyword(native):
    C = native
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(1, 4, 512, 128, device="cuda", generator=g).half()
    k = torch.randn(1, 2, 2048, 128, device="cuda", generator=g).half()
    v = torch.randn(1, 2, 2048, 128, device="cuda", generator=g).half()
    keep = torch.rand(2048, device="cuda", generator=g) > 0.4
    keep[256:1024] = False
    mask = keep[None, None, None, :].expand(1, 4, 512, 2048)
    buf = _buffers(q, k, 128)
    stream = torch.cuda.current_stream().cuda_stream
    tiles = torch.empty(1, 4, 2048 // 128 + 1, dtype=torch.int32, device="cuda")
    C.prepare_key_mask_tiles(cap(mask), cap(tiles), 128, stream)
    out = torch.empty(q.shape, dtype=torch.float16, device="cuda")
    C.risa_sdpa(cap(q), cap(k), cap(v), cap(out), cap(buf["q_int8"]), cap(buf["q_scale"]),
                cap(buf["k_int8"]), cap(buf["k_scale"]), cap(buf["v_int8"]), cap(buf["v_scale"]),
                cap(buf["v_center"]), 128 ** -0.5, 1, 1, True, stream, buf["anchors"].data_ptr(),
                cap(mask), cta_k=128, is_causal=False, key_mask_tiles=cap(tiles))
    want = risa.int8_attention(q, k, v, attn_mask=keep, v_quantization="midpoint_affine")
    assert torch.equal(out, want)


def test_prequantize_attend_construct_reuse_called_like_the_reference(native):
    C = native
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(1, 4, 1000, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 2, 3000, 128, device="cuda", generator=g).bfloat16() * 0.1 + 3
    v = torch.randn(1, 2, 3000, 128, device="cuda", generator=g).bfloat16()
    table = torch.stack([torch.randperm(3000, device="cuda", generator=g) for _ in range(2)])
    table = table.view(1, 2, 3000).int().contiguous()
    buf = _buffers(q, k, 128)
    stream = torch.cuda.current_stream().cuda_stream
    packed = (cap(q), cap(k), cap(v), cap(buf["q_int8"]), cap(buf["q_scale"]), cap(buf["k_int8"]),
              cap(buf["k_scale"]), cap(buf["v_int8"]), cap(buf["v_scale"]), cap(buf["v_center"]),
              128, 2, False, stream, buf["anchors"].data_ptr())
    C.risa_sdpa_quantize(*packed, table.data_ptr())  # fused gather: one table for K and V
    want = risa.prequantize_int8_attention(
        q, k, v, kv_permutation=risa.prepare_kv_permutation(table))
    for ours, ref in ((buf["q_int8"], want.q), (buf["k_int8"], want.k), (buf["v_int8"], want.v),
                      (buf["q_scale"], want.q_scale), (buf["k_scale"], want.k_scale),
                      (buf["v_scale"], want.v_scale), (buf["v_center"], want.v_center)):
        assert torch.equal(ours, ref)

    # without a table, then LSE shift, attention with LSE, capture, selection, sparse reuse
    packed = (cap(q), cap(k), cap(v), cap(buf["q_int8"]), cap(buf["q_scale"]), cap(buf["k_int8"]),
              cap(buf["k_scale"]), cap(buf["v_int8"]), cap(buf["v_scale"]), cap(buf["v_center"]),
              128, 2, False, stream, buf["anchors"].data_ptr())
    C.risa_sdpa_quantize(*packed)
    shift = torch.empty(1, 4, 1000, device="cuda")
    C.risa_lse_shift(cap(q), cap(k), cap(buf["anchors"]), cap(shift), 128 ** -0.5, stream)
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(1, 4, 1000, device="cuda")
    arguments = (cap(buf["q_int8"]), cap(buf["k_int8"]), cap(buf["v_int8"]), cap(out),
                 cap(buf["q_scale"]), cap(buf["k_scale"]), cap(buf["v_scale"]),
                 cap(buf["v_center"]), 128, 128 ** -0.5, 2, stream)
    C.risa_sdpa_prequantized(*arguments, attn_mask=None, sparse_row_offsets=None,
                             sparse_block_indices=None, block_mass=None, is_causal=False,
                             lse=cap(lse))
    want_out, want_lse = risa.int8_attention(q, k, v, return_lse=True)
    assert torch.equal(out, want_out) and torch.equal(lse + shift, want_lse)

    n_q, n_k = 8, 24
    workspace = torch.empty(4 * n_q * n_k + 4 * 1000 * (2 * n_k + 2), device="cuda")
    arguments = (cap(buf["q_int8"]), cap(buf["k_int8"]), cap(buf["v_int8"]), cap(out),
                 cap(buf["q_scale"]), cap(buf["k_scale"]), cap(buf["v_scale"]),
                 cap(buf["v_center"]), 128, 128 ** -0.5, 2, stream)
    C.risa_sdpa_prequantized(*arguments, attn_mask=None, sparse_row_offsets=None,
                             sparse_block_indices=None, block_mass=cap(workspace),
                             is_causal=False, lse=None)
    masses = workspace[: 4 * n_q * n_k].view(-1, n_k)
    rows = masses.shape[0]
    sorted_mass, order = masses.sort(dim=-1, descending=True)
    counts = torch.empty(rows, dtype=torch.int32, device="cuda")
    support = torch.empty_like(masses, dtype=torch.uint8)
    totals = torch.empty(rows, 2, dtype=torch.float64, device="cuda")
    offsets = torch.empty(rows + 1, dtype=torch.int32, device="cuda")
    storage = torch.empty(rows * n_k, dtype=torch.int32, device="cuda")
    summary = torch.empty(3, dtype=torch.float64, device="cuda")
    scan = torch.empty(C.retained_mass_selector_workspace_size(rows), dtype=torch.uint8,
                       device="cuda")
    C.select_retained_mass_csr(cap(sorted_mass), cap(order), cap(counts), cap(support),
                               cap(totals), cap(offsets), cap(storage), cap(summary), cap(scan),
                               0.9, stream)
    selected, total, blocks = summary.tolist()
    _, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.9)
    assert torch.equal(offsets, pattern.row_offsets)
    assert torch.equal(storage[: int(blocks)], pattern.block_indices)
    assert abs(selected / total - pattern.measured_retained_mass) < 1e-12
    arguments = (cap(buf["q_int8"]), cap(buf["k_int8"]), cap(buf["v_int8"]), cap(out),
                 cap(buf["q_scale"]), cap(buf["k_scale"]), cap(buf["v_scale"]),
                 cap(buf["v_center"]), 128, 128 ** -0.5, 2, stream)
    C.risa_sdpa_prequantized(*arguments, attn_mask=None, sparse_row_offsets=cap(offsets),
                             sparse_block_indices=cap(storage[: int(blocks)]), block_mass=None,
                             is_causal=False, lse=None)
    want_sparse = risa.sparse_int8_attention(q, k, v, pattern)
    if pattern.sparsity >= 0.05:
        assert torch.equal(out, want_sparse)


def test_bounded_wait_expires_is_reported_and_the_context_survives():
    """A wait that nothing completes runs out after its limit (1 ms here), the kernel returns, the
    status call names the site, and the next attention call works."""
    C = _backend._C
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    C.device_status()
    C.bounded_wait_self_test(1_000_000, stream)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="site 900"):
        C.device_status()
    C.device_status()  # reading the record clears it
    with pytest.raises(RuntimeError, match="limit"):
        C.bounded_wait_self_test(0, stream)
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(1, 2, 256, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 2, 1500, 128, device="cuda", generator=g).bfloat16()
    out = risa.int8_attention(q, k, k)
    torch.cuda.synchronize()
    C.device_status()
    assert torch.isfinite(out.float()).all()
