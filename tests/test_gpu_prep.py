"""Q/K/V preparation kernels against the reference's own kernels: every code, scale, anchor and
centre must be bit-identical."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.util import qkv  # noqa: E402


def _ours(q, k, v, cta_k, affine):
    from risaattention_b200 import _backend
    from risaattention_b200._quantization import PackedBuffers, quantize_into

    buf = PackedBuffers(q, k, cta_k)
    quantize_into(buf, q, k, v, cta_k, affine)
    return buf


def _centers_match(ours, want):
    """Midpoint-affine centres: bit-identical except for rare channels one ulp away."""
    ulp = torch.nextafter(want.abs(), torch.full_like(want, 9e9)) - want.abs()
    assert ((ours - want).abs() <= ulp).all()
    assert (ours != want).float().mean() < 0.01


CASES = [
    # d, lq, lk, cta_k, hq, hkv
    (64, 137, 200, 64, 4, 2),      # H4 rotation (Lk <= 256), partial blocks
    (64, 300, 1025, 64, 4, 4),     # H64
    (128, 137, 263, 64, 2, 1),     # signed H128, 64-key tiles
    (128, 257, 1153, 128, 4, 2),   # 128-key tiles, ragged tail
    (128, 1024, 2048, 128, 8, 2),
    (256, 137, 263, 64, 2, 1),     # plain H128 per half
    (256, 200, 1153, 128, 4, 2),
    (128, 100, 100, 64, 2, 2),     # H4 with D128
    (256, 33, 64, 64, 2, 1),
    (128, 128, 8192, 128, 2, 1),   # tiled V code pass, 16 windows per slot
    (64, 64, 16400, 64, 2, 2),     # ... 33 windows, the last one short
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("anchor", [False, True])
def test_prep_bit_exact(ref, dtype, case, anchor):
    d, lq, lk, cta_k, hq, hkv = case
    for affine in (False, True):
        q, k, v = qkv(2, hq, hkv, lq, lk, d, dtype, seed=lq + lk, anchor=anchor)
        v = v + 1.5
        got = _ours(q, k, v, cta_k, affine)
        want = ref.prequantize(q, k, v, cta_k=cta_k, midpoint_affine=affine)
        torch.cuda.synchronize()
        assert torch.equal(got.anchors, want["anchors"])
        if anchor:
            assert (want["anchors"] >= 0).any(), "test data was meant to trigger the anchor"
        assert torch.equal(got.q_codes, want["q"])
        assert torch.equal(got.k_codes, want["k"])
        assert torch.equal(got.q_scales, want["q_scale"])
        assert torch.equal(got.k_scales, want["k_scale"])
        assert torch.equal(got.v_codes, want["v"])
        assert torch.equal(got.v_scales, want["v_scale"])
        _centers_match(got.v_centers, want["v_center"])


@pytest.mark.parametrize("layout", ["nhd"])
def test_prep_strided_inputs(ref, layout):
    q, k, v = qkv(2, 4, 2, 300, 1500, 128, torch.bfloat16, seed=5, layout=layout)
    got = _ours(q, k, v, 128, True)
    want = ref.prequantize(q, k, v, cta_k=128, midpoint_affine=True)
    for a, b in ((got.q_codes, want["q"]), (got.k_codes, want["k"]), (got.v_codes, want["v"]),
                 (got.q_scales, want["q_scale"]), (got.v_scales, want["v_scale"])):
        assert torch.equal(a, b)
    _centers_match(got.v_centers, want["v_center"])


def test_prep_against_cpu_oracle():
    """Second opinion: the CPU restatement agrees up to its documented budget (approximate
    division / reciprocal cannot be reproduced on a CPU): codes differ by at most 1, rarely."""
    from oracle import risa_oracle as O

    q, k, v = qkv(1, 4, 2, 300, 1153, 128, torch.bfloat16, seed=3)
    got = _ours(q, k, v, 128, True)
    anchors = O.detect_k_anchor(k.float().cpu())
    assert torch.equal(anchors, got.anchors.cpu())
    qc, qs = O.quantize_q(q.float().cpu(), 1153)
    kc, ks = O.quantize_k(k.float().cpu(), 128, anchors)
    vc, vs, vcen = O.quantize_v(v.float().cpu(), 128, True)
    for mine, oracle in ((got.q_codes, qc), (got.k_codes, kc), (got.v_codes, vc)):
        diff = (mine.cpu().int() - oracle.int()).abs()
        assert diff.max() <= 1 and (diff > 0).float().mean() < 2e-3
    torch.testing.assert_close(got.q_scales.cpu(), qs, rtol=1e-6, atol=0)
    torch.testing.assert_close(got.k_scales.cpu(), ks, rtol=1e-6, atol=0)
    torch.testing.assert_close(got.v_scales.cpu(), vs, rtol=1e-6, atol=0)
    # a code that differs by one moves the centre by scale / Lk
    torch.testing.assert_close(got.v_centers.cpu(), vcen, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", ["hnd", "nhd", "interleaved"])
@pytest.mark.parametrize("length", [1025, 2048, 2049, 4097])
def test_absmax_values_known_answer(dtype, length, layout):
    """Power-of-two data make codes and scales independent of rounding (the reference's own
    known-answer test, tests/cuda/test_value_quantization.py:18-52), for head-major, token-major
    and fused-QKV storage of V."""
    import risaattention_b200 as risa

    batch, heads, channels = 2, 3, 128
    tokens = torch.arange(length, device="cuda")[None, None, :, None]
    offs = torch.arange(batch * heads, device="cuda").reshape(batch, heads, 1, 1)
    codes = ((tokens + offs) % 255 - 127).expand(batch, heads, length, channels)
    scales = 2.0 ** ((torch.arange(channels, device="cuda") % 4).float() - 2)
    v = (codes * scales).to(dtype)
    if layout == "nhd":
        v = v.transpose(1, 2).contiguous().transpose(1, 2)
    elif layout == "interleaved":
        fused = torch.empty(batch, length, 3, heads, channels, device="cuda", dtype=dtype)
        v = fused[:, :, 1].transpose(1, 2).copy_(v)
    q = torch.zeros(batch, heads * 2, 3, channels, device="cuda", dtype=dtype)
    packed = risa.prequantize_int8_attention(q, torch.zeros_like(v), v, v_quantization="absmax")
    padded = packed.v.shape[-1]
    expected = torch.zeros(batch, heads, channels, padded, device="cuda", dtype=torch.int8)
    expected[..., :length] = codes.transpose(2, 3).to(torch.int8)
    order = torch.tensor([0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15], device="cuda")
    expected = expected.reshape(batch, heads, channels, -1, 16)[..., order]
    assert torch.equal(packed.v.reshape_as(expected), expected)
    assert torch.equal(packed.v_scale.reshape(batch, heads, channels),
                       scales.expand(batch, heads, channels))
    assert torch.count_nonzero(packed.v_center) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("dim", [64, 128, 256])
def test_lse_shift(ref, dtype, dim):
    from risaattention_b200 import _backend

    torch.manual_seed(35)
    q = torch.randn(2, 17, 4, dim, device="cuda", dtype=dtype).transpose(1, 2)
    k = torch.randn(2, 9, 2, dim, device="cuda", dtype=dtype).transpose(1, 2)
    anchors = torch.tensor([[-1, 0], [3, 2]], device="cuda", dtype=torch.int32)
    out = torch.empty(2, 4, 17, device="cuda")
    _backend._C.risa_lse_shift(q, k, anchors, out, dim ** -0.5,
                               torch.cuda.current_stream().cuda_stream)
    assert torch.equal(out, ref.lse_shift(q, k, anchors, dim ** -0.5))
    sel = k.gather(2, anchors.clamp_min(0).long()[..., None, None].expand(2, 2, 1, dim))
    sel = sel.float() * (anchors >= 0)[..., None, None]
    expect = (q.float() * sel.repeat_interleave(2, 1)).sum(-1) * dim ** -0.5
    torch.testing.assert_close(out, expect, rtol=2e-5, atol=5e-6)
    assert torch.count_nonzero(out[0, :2]) == 0


@pytest.mark.parametrize("dim", [32, 96, 8])
@pytest.mark.parametrize("lk", [64, 1040, 333])
@pytest.mark.parametrize("affine", [False, True])
def test_quantize_v_c_abi_head_dims_outside_the_kernel_set(ref, dim, lk, affine):
    """The C-ABI accepts any head_dim that is a multiple of 8 (the Python runtime only ever passes
    64 / 128 / 256): such sizes must take the channel-generic kernels, also when the key length is
    a multiple of 16, and match the reference's kernel bit for bit."""
    import ctypes

    from oracle import ref_gpu
    from risaattention_b200 import _backend

    b, hkv = 2, 3
    g = torch.Generator(device="cuda").manual_seed(dim + lk)
    v = (torch.randn(b, hkv, lk, dim, device="cuda", generator=g) + 0.7).bfloat16()
    padded = -(-lk // 64) * 64
    channels = b * hkv * dim
    stream = torch.cuda.current_stream().cuda_stream

    def buffers():
        return (torch.full((channels, padded), 77, dtype=torch.int8, device="cuda"),
                torch.empty(channels, device="cuda"), torch.empty(channels, device="cuda"))

    codes, scale, center = buffers()
    C = _backend._ABI
    ws = torch.empty(C.quantize_v_workspace_size(b, hkv, lk, dim), dtype=torch.uint8, device="cuda")
    guard = torch.zeros(4096, dtype=torch.uint8, device="cuda")  # allocated right after the outputs
    C._check(C.lib.risa_b200_quantize_v(
        ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(codes.data_ptr()),
        ctypes.c_void_p(scale.data_ptr()), ctypes.c_void_p(center.data_ptr()), b, hkv, lk, dim,
        padded, v.stride(0), v.stride(1), v.stride(2), 2, int(affine), None,
        ctypes.c_void_p(ws.data_ptr()), ws.numel(), stream))
    rc, rs, rcen = buffers()
    ref_gpu._ok(ref_gpu.lib().ref_quantize_v(
        ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(rc.data_ptr()),
        ctypes.c_void_p(rs.data_ptr()), ctypes.c_void_p(rcen.data_ptr()), b, hkv, lk, dim, padded,
        v.stride(0), v.stride(1), v.stride(2), 2, int(affine), stream))
    torch.cuda.synchronize()
    assert torch.equal(codes, rc) and torch.equal(scale, rs)
    _centers_match(center, rcen)
    assert int(guard.sum()) == 0


@pytest.mark.parametrize("case", [CASES[0], CASES[3], CASES[6]])
@pytest.mark.parametrize("affine", [False, True])
def test_separate_entry_points_equal_the_combined_call(case, affine):
    """risa_b200_quantize_qk + risa_b200_quantize_v (anchor detector, range pass and Q quantiser as
    launches of their own) give the bytes of risa_b200_quantize_qkv (one launch for the three)."""
    import ctypes

    from risaattention_b200 import _backend
    from risaattention_b200._quantization import PackedBuffers

    d, lq, lk, cta_k, hq, hkv = case
    q, k, v = qkv(2, hq, hkv, lq, lk, d, torch.bfloat16, seed=7 + lq, anchor=True)
    v = v + 0.75
    combined = _ours(q, k, v, cta_k, affine)
    apart = PackedBuffers(q, k, cta_k)
    C = _backend._ABI
    stream = torch.cuda.current_stream().cuda_stream
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    b = q.shape[0]
    C._check(C.lib.risa_b200_quantize_qk(
        p(q), p(apart.q_codes), p(apart.q_scales), p(k), p(apart.k_codes), p(apart.k_scales), b, hq,
        lq, hkv, lk, d, cta_k, q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1),
        k.stride(2), 2, p(apart.anchors), None, None, stream))
    C._check(C.lib.risa_b200_quantize_v(
        p(v), p(apart.v_codes), p(apart.v_scales), p(apart.v_centers), b, hkv, lk, d,
        apart.v_codes.shape[1], v.stride(0), v.stride(1), v.stride(2), 2, int(affine), None,
        p(apart.workspace), apart.workspace.numel(), stream))
    torch.cuda.synchronize()
    for name in ("anchors", "q_codes", "q_scales", "k_codes", "k_scales", "v_codes", "v_scales",
                 "v_centers"):
        assert torch.equal(getattr(combined, name), getattr(apart, name)), name


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_quantisation_on_a_side_stream_and_in_a_graph(mode):
    """Quantising on a stream other than the default one, and replaying the same call from a
    captured graph, gives the bytes of the plain call (reference behaviour:
    tests/cuda/test_value_quantization.py:75-91); the chained launches of the call are captured
    with their programmatic dependencies."""
    import risaattention_b200 as risa

    g = torch.Generator(device="cuda").manual_seed(75)
    q = torch.randn(1, 4, 17, 128, device="cuda", generator=g).bfloat16()
    k, v = [torch.randn(1, 2, 4097, 128, device="cuda", generator=g).bfloat16() for _ in range(2)]
    plain = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        expected = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            actual = risa.prequantize_int8_attention(q, k, v, v_quantization=mode)
        for name in ("q", "k", "v", "q_scale", "k_scale", "v_scale", "v_center"):
            getattr(actual, name).zero_()
        graph.replay()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    for name in ("q", "k", "v", "q_scale", "k_scale", "v_scale", "v_center"):
        assert torch.equal(getattr(actual, name), getattr(expected, name)), name
        assert torch.equal(getattr(plain, name), getattr(expected, name)), name
