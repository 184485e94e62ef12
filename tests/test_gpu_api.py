"""Public API behaviour on the GPU: the reference's own known-answer and contract tests
(tests/cuda/test_risa_attention.py, test_probability_mass.py, test_key_mask_tiles.py) restated
against this package, plus accuracy against FP32 SDPA."""
from dataclasses import replace

import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200._validation import apply_score_mask  # noqa: E402
from tests.util import assert_outputs_match, nrmse  # noqa: E402


def test_available():
    assert risa.int8_attention_is_available()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("key_length", [512, 1025])
@pytest.mark.parametrize("scale", [None, 0.0, -0.125])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_constant_values_preserve_probability_mass(dtype, head_dim, key_length, scale, mode):
    torch.manual_seed(41)
    q = torch.randn(1, 4, 129, head_dim, device="cuda", dtype=dtype)
    k = torch.randn(1, 2, key_length, head_dim, device="cuda", dtype=dtype)
    values = torch.linspace(-3, 5, head_dim, device="cuda", dtype=dtype)
    v = values.expand_as(k).contiguous()
    out = risa.int8_attention(q, k, v, scale=scale, v_quantization=mode)
    assert torch.equal(out, values.expand_as(out))


@pytest.mark.parametrize("key_length", [512, 1025])
@pytest.mark.parametrize("scale", [0.0, -0.125])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_signed_scale_tail_masks_and_lse(key_length, scale, mode):
    torch.manual_seed(43)
    q = torch.randn(1, 4, 129, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 2, key_length, 128, device="cuda", dtype=q.dtype)
    v = torch.full_like(k, 3)
    mask = torch.ones(129, key_length, device="cuda", dtype=torch.bool)
    mask[0] = False
    mask[1:, 7::9] = False
    out, lse = risa.int8_attention(q, k, v, scale=scale, attn_mask=mask, is_causal=True,
                                   v_quantization=mode, return_lse=True)
    assert torch.equal(out[:, :, 1:], torch.full_like(out[:, :, 1:], 3))
    assert torch.count_nonzero(out[:, :, 0]) == 0
    assert torch.isneginf(lse[:, :, 0]).all() and torch.isfinite(lse[:, :, 1:]).all()
    if scale == 0:
        visible = mask & (torch.arange(key_length, device="cuda")[None, :]
                          <= torch.arange(129, device="cuda")[:, None])
        torch.testing.assert_close(lse, visible.sum(-1).float().log().expand_as(lse), atol=2e-5,
                                   rtol=0)


def test_residual_center_preserves_uniform_attention_mean():
    q = torch.zeros(1, 2, 129, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 1, 512, 128, device="cuda", dtype=q.dtype)
    torch.manual_seed(1)
    v = torch.randn_like(k) + 3
    v[..., ::53, :] += 12
    out = risa.int8_attention(q, k, v, v_quantization="midpoint_affine")
    assert torch.equal(out, v.float().mean(-2, keepdim=True).to(v.dtype).expand_as(out))


@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("length", [63, 65, 193, 1153])
@pytest.mark.parametrize("mode", ["midpoint_affine", "absmax"])
def test_capture_tile_max_known_answer(dim, length, mode):
    """Hand-filled packed operands pin the captured tile maxima to
    float(level * D * log2(e) / 128 - 7.9943534), capture must not change output bits, and a fully
    masked call returns exact zeros (reference tests/cuda/test_risa_attention.py:20-92)."""
    q = torch.zeros(1, 2, 137, dim, device="cuda", dtype=torch.float16)
    k = torch.zeros(1, 1, length, dim, device="cuda", dtype=torch.float16)
    torch.manual_seed(2)
    packed = risa.prequantize_int8_attention(q, k, torch.randn_like(k) + 2, scale=1 / 128,
                                             v_quantization=mode)
    packed.q.fill_(1)
    packed.q_scale.fill_(1)
    packed.k_scale.fill_(1)
    blocks = -(-length // packed.cta_k)
    levels = torch.tensor([3 if i % 2 == 0 else -2 for i in range(blocks)], dtype=torch.int8,
                          device="cuda")
    for i in range(blocks):
        packed.k[:, :, i * packed.cta_k:(i + 1) * packed.cta_k].fill_(3 if i % 2 == 0 else -2)
    b, h, n, _ = packed.q.shape
    mass_elements = b * h * ((n + 127) // 128) * blocks
    rows = b * h * n
    ws = torch.empty(mass_elements + rows * (blocks * 2 + 2), device="cuda")
    plain = risa.int8_attention_from_prequantized(packed)
    captured = risa.int8_attention_from_prequantized(packed, _block_mass=ws)
    assert torch.equal(plain.view(torch.int16), captured.view(torch.int16))
    if blocks > 1:
        maxima = ws[mass_elements:mass_elements + rows * (blocks - 1) * 2].reshape(
            rows, blocks - 1, 2)[..., 1]
        scale = torch.tensor(1.44269504088896340736, device="cuda") / 128
        offset = torch.tensor(7.9943534, device="cuda")
        expected = (levels[:-1].double() * dim * scale.double() - offset.double()).float()
        assert torch.equal(maxima, expected.expand_as(maxima))
    hidden = torch.zeros(b, h, n, length, device="cuda", dtype=torch.bool)
    empty = risa.int8_attention_from_prequantized(replace(packed, attn_mask=hidden))
    assert torch.count_nonzero(empty.view(torch.int16)) == 0


@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("mode", ["midpoint_affine", "absmax"])
def test_dense_sparse_causal_masks_and_v_modes(dim, mode):
    torch.manual_seed(17)
    q = torch.randn(1, 2, 137, dim, device="cuda", dtype=torch.float16)
    k = torch.randn(1, 1, 263, dim, device="cuda", dtype=torch.float16)
    v = torch.randn_like(k) + 2
    key_bias = torch.linspace(-2, 0, 263, device="cuda")[None, None, None, :]
    row_mask = torch.ones(137, 263, device="cuda", dtype=torch.bool)
    row_mask[0] = False
    for causal in (False, True):
        for mask in (None, key_bias, row_mask):
            opts = dict(v_quantization=mode, is_causal=causal, attn_mask=mask)
            dense = risa.int8_attention(q, k, v, **opts)
            built, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=1.0, **opts)
            sparse = risa.sparse_int8_attention(q, k, v, pattern, **opts)
            packed = risa.prequantize_int8_attention(q, k, v, **opts)
            split = risa.int8_attention_from_prequantized(packed, sparse_pattern=pattern,
                                                          output_layout="nhd")
            scores = q.float() @ k.float().repeat_interleave(2, 1).transpose(-1, -2) / dim ** 0.5
            expanded = None if mask is None else torch.broadcast_to(mask, scores.shape)
            scores = apply_score_mask(scores, expanded, causal, 0)
            want = scores.softmax(-1).nan_to_num(nan=0) @ v.float().repeat_interleave(2, 1)
            torch.testing.assert_close(dense.float(), want, atol=0.10, rtol=0.03)
            torch.testing.assert_close(built, dense, atol=0.03, rtol=0.01)
            torch.testing.assert_close(sparse, dense, atol=0.04, rtol=0.01)
            torch.testing.assert_close(split, sparse, atol=0.005, rtol=0.005)
            if mask is row_mask:
                assert sparse[:, :, 0].count_nonzero().item() == 0
            if mode == "absmax":
                assert packed.v_center.count_nonzero().item() == 0
            with pytest.raises(ValueError, match="is_causal"):
                risa.sparse_int8_attention(q, k, v, pattern, v_quantization=mode, attn_mask=mask,
                                           is_causal=not causal)


def test_lse_restores_shifted_keys_and_empty_rows():
    torch.manual_seed(29)
    q = torch.randn(1, 2, 19, 128, device="cuda", dtype=torch.float16)
    k = torch.randn(1, 1, 257, 128, device="cuda", dtype=torch.float16) * 0.1 + 4
    v = torch.randn_like(k)
    mask = torch.ones(19, 257, dtype=torch.bool, device="cuda")
    mask[0] = False
    out, lse = risa.int8_attention(q, k, v, attn_mask=mask, is_causal=True, return_lse=True)
    scores = q.float() @ k.float().transpose(-1, -2) / 128 ** 0.5
    want = apply_score_mask(scores, mask, True, 0).logsumexp(-1)
    assert torch.isneginf(lse[:, :, 0]).all()
    assert out[:, :, 0].count_nonzero().item() == 0
    torch.testing.assert_close(lse[:, :, 1:], want[:, :, 1:], atol=0.15, rtol=0.02)


def test_key_mask_metadata_and_skipping():
    from risaattention_b200._key_mask import prepare_key_mask_tiles

    torch.manual_seed(3)
    q = torch.randn(1, 4, 257, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 2, 1153, 128, device="cuda", dtype=q.dtype)
    v = torch.randn_like(k)
    mask = torch.ones(1, 1, 1, 1153, device="cuda", dtype=torch.bool)
    mask[..., :512] = False
    packed = risa.prequantize_int8_attention(q, k, v, attn_mask=mask)
    tiles = prepare_key_mask_tiles(packed.attn_mask, packed.cta_k, 257, packed.attention_scale,
                                   False)
    expected = torch.tensor([4, 5, 6, 7, 8, 9], device="cuda", dtype=torch.int32)
    assert torch.equal(tiles[..., :6], expected.expand(1, 4, 6))
    assert (tiles[..., -1] == 6).all()
    actual = risa.int8_attention_from_prequantized(packed)
    generic = risa.int8_attention_from_prequantized(
        replace(packed, attn_mask=packed.attn_mask.clone()))
    torch.testing.assert_close(actual, generic, atol=0.002, rtol=0.01)


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_key_mask_is_read_at_call_time(mode):
    """The visible-tile list of a broadcast key mask is rebuilt by every call, inside a captured
    graph as well: a mask changed in place after prequantisation (or between replays) is the mask
    the next call sees (reference behaviour: tests/cuda/test_key_mask_tiles.py:79-128)."""
    g = torch.Generator(device="cuda").manual_seed(21)
    q = torch.randn(1, 4, 300, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 2, 1300, 128, device="cuda", generator=g).bfloat16()
    v = torch.full_like(k, 1.5)
    mask = torch.ones(1, 1, 1, 1300, device="cuda", dtype=torch.bool)
    mask[..., :640] = False
    packed = risa.prequantize_int8_attention(q, k, v, attn_mask=mask, v_quantization=mode)
    hidden_prefix = risa.int8_attention_from_prequantized(packed)
    mask.fill_(True)  # in place: `packed` holds the same storage
    all_visible = risa.int8_attention_from_prequantized(packed)
    fresh = risa.int8_attention_from_prequantized(
        risa.prequantize_int8_attention(q, k, v, attn_mask=mask.clone(), v_quantization=mode))
    assert torch.equal(all_visible, fresh)
    assert torch.allclose(hidden_prefix.float(), all_visible.float(), atol=0.02)  # V is constant
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            risa.int8_attention_from_prequantized(packed)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = risa.int8_attention_from_prequantized(packed)
        mask.fill_(False)  # every key hidden: rows must come out as zeros
        graph.replay()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    assert torch.count_nonzero(captured) == 0


@pytest.mark.parametrize("length", [512, 2048])
@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_accuracy_against_fp32_sdpa(length, mode):
    """NRMSE against FP32 SDPA stays at the reference's published level (0.0145-0.0158 for these
    lengths, README.md:117-119) plus 5 %."""
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(1, 16, length, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 4, length, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(1, 4, length, 128, device="cuda", generator=g).bfloat16()
    out = risa.int8_attention(q, k, v, v_quantization=mode)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(4, 1), v.float().repeat_interleave(4, 1))
    assert nrmse(out, want) <= 0.0160 * 1.05


def test_graph_capture_and_streams():
    q = torch.randn(1, 4, 300, 128, device="cuda", dtype=torch.bfloat16)
    k, v = [torch.randn(1, 2, 1500, 128, device="cuda", dtype=q.dtype) for _ in range(2)]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        expected = risa.int8_attention(q, k, v, v_quantization="midpoint_affine")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            actual = risa.int8_attention(q, k, v, v_quantization="midpoint_affine")
        graph.replay()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    assert torch.equal(actual, expected)


def test_graph_replays_follow_their_inputs():
    """A captured dense call (chained launches, split last wave and merge launch included) replayed
    after its inputs were overwritten in place gives what an eager call gives on the new inputs."""
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(1, 16, 4096, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 4, 4096, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(1, 4, 4096, 128, device="cuda", generator=g).bfloat16()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            risa.int8_attention(q, k, v)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = risa.int8_attention(q, k, v)
        for _ in range(3):
            q.copy_(torch.randn(q.shape, device="cuda", generator=g).bfloat16())
            k.copy_(torch.randn(k.shape, device="cuda", generator=g).bfloat16())
            v.copy_(torch.randn(v.shape, device="cuda", generator=g).bfloat16())
            graph.replay()
            replayed = captured.clone()
            eager = risa.int8_attention(q, k, v)
            assert torch.equal(replayed, eager)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()


def test_host_pipeline_matches_device_call():
    """Host-resident operands, pipelined per KV head over three streams: identical bits to one
    device-resident call (every stage is independent per head)."""
    import risaattention_b200 as risa

    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 8, 300, 128, generator=g).bfloat16().pin_memory()
    k = torch.randn(2, 2, 1300, 128, generator=g).bfloat16().pin_memory()
    v = torch.randn(2, 2, 1300, 128, generator=g).bfloat16().pin_memory()
    for causal in (False, True):
        want = risa.int8_attention(q.cuda(), k.cuda(), v.cuda(), is_causal=causal,
                                   v_quantization="midpoint_affine")
        got = risa.int8_attention_from_host(q, k, v, is_causal=causal,
                                            v_quantization="midpoint_affine")
        torch.cuda.synchronize()
        assert got.is_pinned() and torch.equal(got, want.cpu())
    with pytest.raises(ValueError, match="does not support"):
        risa.int8_attention_from_host(q, k, v, return_lse=True)


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_causal_rows_never_see_later_values(mode):
    """Values that only exist at later positions cannot reach earlier causal rows, dense or through
    a retained pattern (reference behaviour: tests/cuda/test_risa_attention.py:151-165)."""
    q = torch.zeros(1, 1, 200, 64, device="cuda", dtype=torch.float16)
    v = torch.zeros_like(q)
    v[:, :, 128:] = 64.0
    dense, pattern = risa.construct_sparse_int8_attention(q, q, v, is_causal=True, theta=1.0,
                                                          v_quantization=mode)
    sparse = risa.sparse_int8_attention(q, q, v, pattern, is_causal=True, v_quantization=mode)
    assert dense[:, :, :128].abs().max() <= 0.01
    assert dense[:, :, 199].float().mean() > 10  # the last row sees 72 of 200 non-zero values
    torch.testing.assert_close(sparse, dense, atol=0.05, rtol=0.01)


@pytest.mark.parametrize("mode", ["absmax", "midpoint_affine"])
def test_key_bias_with_large_tiles_and_lse(mode):
    """A float mask broadcast over queries keeps 128-key tiles; with zero scores the output is the
    constant value and the LSE is the log-sum-exp of the bias (reference behaviour:
    tests/cuda/test_risa_attention.py:167-179)."""
    q = torch.zeros(1, 2, 17, 128, device="cuda", dtype=torch.float16)
    k = torch.zeros(1, 1, 1200, 128, device="cuda", dtype=torch.float16)
    v = torch.full_like(k, 2.5)
    bias = torch.linspace(-4, 0, 1200, device="cuda")[None, None, None, :]
    packed = risa.prequantize_int8_attention(q, k, v, attn_mask=bias, return_lse=True,
                                             v_quantization=mode)
    assert packed.cta_k == 128
    out, lse = risa.int8_attention_from_prequantized(packed, return_lse=True)
    assert (out.float() - 2.5).abs().max() <= 0.03
    want = bias.logsumexp(-1).expand(1, 2, 17)
    assert (lse - want).abs().max() <= 0.01


def test_packed_value_rows_beyond_two_gibibytes():
    """56 heads x 128 channels of 299 521 keys: the packed V tensor is 2.15 GB, so element offsets
    into it do not fit 32 bits (the reference keeps this as an opt-in large test:
    tests/cuda/test_risa_attention.py:195-208).  Constant values must come back exactly."""
    if torch.cuda.mem_get_info()[0] < 24 * 1024 ** 3:
        pytest.skip("needs 24 GiB of free device memory")
    heads, keys = 56, 299521
    q = torch.zeros(1, heads, 1, 128, device="cuda", dtype=torch.float16)
    k = torch.zeros(1, heads, keys, 128, device="cuda", dtype=torch.float16)
    v = torch.ones_like(k)
    v[:, -1] = 3.0  # the last head's rows lie wholly beyond the 2 GiB mark
    for mode in ("absmax", "midpoint_affine"):
        out = risa.int8_attention(q, k, v, v_quantization=mode)
        torch.cuda.synchronize()
        assert (out[:, :-1].float() - 1.0).abs().max() <= 0.01
        assert (out[:, -1].float() - 3.0).abs().max() <= 0.03
        del out
    del q, k, v
    torch.cuda.empty_cache()


@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("key_length", [1, 5, 17, 63, 64, 65, 127, 128])
@pytest.mark.parametrize("is_causal", [False, True])
def test_key_sequences_of_one_or_two_tiles(head_dim, key_length, is_causal):
    """Fewer keys than one tile, exactly one tile, and one key more: the packed V row is shorter
    than the 128-key slab the tensor-core kernel loads up to 64 keys (those calls take the
    row-per-thread kernel), and a single tile is first and last at once.  Against the FP32
    specification; with one key the output is that key's value whatever the scores are."""
    from risaattention_b200 import _backend

    g = torch.Generator(device="cuda").manual_seed(100 * head_dim + key_length)
    q = torch.randn(1, 4, 200, head_dim, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 2, key_length, head_dim, device="cuda", generator=g).bfloat16()
    v = torch.randn(1, 2, key_length, head_dim, device="cuda", generator=g).bfloat16()
    scores = q.float() @ k.float().repeat_interleave(2, 1).transpose(-1, -2) / head_dim ** 0.5
    scores = apply_score_mask(scores, None, is_causal, 0)
    want = scores.softmax(-1) @ v.float().repeat_interleave(2, 1)
    outputs = []
    for path in (0, 1):
        previous = _backend._C.set_attention_path(path)
        try:
            out, lse = risa.int8_attention(q, k, v, is_causal=is_causal, return_lse=True,
                                           v_quantization="midpoint_affine")
        finally:
            _backend._C.set_attention_path(previous)
        _backend._C.device_status()
        outputs.append(out)
        assert nrmse(out, want) <= 0.04
        torch.testing.assert_close(lse, scores.logsumexp(-1), atol=0.15, rtol=0.02)
        if key_length == 1:
            step = v.float().abs().amax() / 127
            assert (out.float() - v.float().repeat_interleave(2, 1)).abs().max() <= step
    assert_outputs_match(outputs[0], outputs[1], 2e-3)


def test_concurrent_host_threads_on_their_own_streams():
    """Four host threads, each on a stream of its own, interleave dense, masked, LSE and pattern
    calls; every result equals the one the same call gives alone (per-call scratch, thread-local
    error text and launch configuration, no state shared between calls)."""
    import threading

    def inputs(seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        q = torch.randn(1, 4, 260 + 16 * seed, 128, device="cuda", generator=g).bfloat16()
        k = torch.randn(1, 2, 1100 + 64 * seed, 128, device="cuda", generator=g).bfloat16()
        v = torch.randn(1, 2, 1100 + 64 * seed, 128, device="cuda", generator=g).bfloat16()
        return q, k, v

    def routes(q, k, v):
        mask = torch.ones(1, 1, 1, k.shape[2], dtype=torch.bool, device="cuda")
        mask[..., ::3] = False
        dense = risa.int8_attention(q, k, v, v_quantization="midpoint_affine")
        out, lse = risa.int8_attention(q, k, v, is_causal=True, return_lse=True)
        masked = risa.int8_attention(q, k, v, attn_mask=mask)
        built, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.9)
        sparse = risa.sparse_int8_attention(q, k, v, pattern)
        return [dense, out, lse, masked, built, sparse, pattern.block_indices]

    cases = [inputs(seed) for seed in range(4)]
    alone = [routes(*case) for case in cases]
    torch.cuda.synchronize()
    results, failures = [None] * 4, []

    def worker(index):
        try:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.default_stream())
            with torch.cuda.stream(stream):
                for _ in range(5):
                    results[index] = routes(*cases[index])
            stream.synchronize()
        except Exception as error:  # noqa: BLE001 - reported by the main thread
            failures.append((index, error))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures
    from risaattention_b200 import _backend

    _backend._C.device_status()
    for got, want in zip(results, alone):
        for a, b in zip(got, want):
            assert torch.equal(a, b)
