"""The tensor-core attention kernel is compiled once per class of call (no mask / causal / boolean
per-query masks read as bits / other per-query masks / masks broadcast over the queries), each
instantiation holding only the softmax paths its calls take.  Every class must give the bits of the
instantiation that holds all paths (``set_attention_path(2)``, a per-thread diagnostic switch)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import _backend  # noqa: E402


def _inputs(head_dim, q_len, k_len, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(2, 4, q_len, head_dim, device="cuda", generator=g).bfloat16()
    k = torch.randn(2, 2, k_len, head_dim, device="cuda", generator=g).bfloat16()
    v = torch.randn(2, 2, k_len, head_dim, device="cuda", generator=g).bfloat16() + 0.5
    return q, k, v, g


def _masks(kind, q_len, k_len, g):
    if kind == "bool_rows":
        mask = torch.rand(2, 4, q_len, k_len, device="cuda", generator=g) > 0.4
        mask[:, :, 3] = False  # an empty row
        return mask
    if kind == "bool_rows_shared_over_heads":
        return (torch.rand(2, 1, q_len, k_len, device="cuda", generator=g) > 0.4)
    if kind == "fp32_bias":
        return torch.randn(2, 4, q_len, k_len, device="cuda", generator=g)
    if kind == "fp16_bias":
        return torch.randn(2, 4, q_len, k_len, device="cuda", generator=g).half()
    if kind == "key_bias":
        bias = torch.randn(2, 1, 1, k_len, device="cuda", generator=g)
        bias[..., ::11] = float("-inf")
        return bias
    if kind == "key_bias_bf16":
        return torch.randn(1, 1, 1, k_len, device="cuda", generator=g).bfloat16()
    if kind == "key_bool":
        keep = torch.ones(2, 1, 1, k_len, device="cuda", dtype=torch.bool)
        keep[..., : k_len // 3] = False
        keep[..., ::5] = False
        return keep
    return None


def _both(call):
    results = []
    for path in (0, 2):
        previous = _backend._C.set_attention_path(path)
        try:
            results.append(call())
        finally:
            _backend._C.set_attention_path(previous)
    torch.cuda.synchronize()
    _backend._C.device_status()
    return results


@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("k_len", [1300, 1024, 700])
@pytest.mark.parametrize("kind", ["plain", "causal", "bool_rows", "bool_rows_shared_over_heads",
                                  "fp32_bias", "fp16_bias", "key_bias", "key_bias_bf16",
                                  "key_bool", "bool_rows+causal", "key_bias+causal"])
def test_class_kernels_give_the_bits_of_the_all_paths_kernel(head_dim, k_len, kind):
    q, k, v, g = _inputs(head_dim, 300, k_len, seed=head_dim + k_len)
    mask = _masks(kind.split("+")[0], 300, k_len, g)
    causal = kind == "causal" or kind.endswith("+causal")
    for mode in ("absmax", "midpoint_affine"):
        own, every = _both(lambda: risa.int8_attention(q, k, v, attn_mask=mask, is_causal=causal,
                                                       return_lse=True, v_quantization=mode))
        assert torch.equal(own[0], every[0])
        assert torch.equal(own[1].view(torch.int32), every[1].view(torch.int32))
    if kind == "bool_rows":
        assert own[0][:, :, 3].count_nonzero() == 0 and torch.isneginf(own[1][:, :, 3]).all()


@pytest.mark.parametrize("head_dim", [64, 128])
def test_class_kernels_in_pattern_construction_and_reuse(head_dim):
    """Capture, in-pass selection and sparse reuse of calls without mask or causal rule run in the
    instantiations of that class: same outputs, same tile sets."""
    q, k, v, _ = _inputs(head_dim, 1500, 1500, seed=9)

    def construct():
        return risa.construct_sparse_int8_attention(q, k, v, theta=0.9)

    (out_a, pat_a), (out_b, pat_b) = _both(construct)
    assert torch.equal(out_a, out_b)
    assert torch.equal(pat_a.row_offsets, pat_b.row_offsets)
    assert torch.equal(pat_a.block_indices, pat_b.block_indices)
    assert pat_a.measured_retained_mass == pat_b.measured_retained_mass
    reuse_a, reuse_b = _both(lambda: risa.sparse_int8_attention(q, k, v, pat_a))
    assert torch.equal(reuse_a, reuse_b)
    # the reference's route (capture workspace, block-mass kernel, library sort, selector)
    packed = risa.prequantize_int8_attention(q, k, v)
    from risaattention_b200._execution import capture_workspace_elements

    def capture():
        workspace = torch.zeros(capture_workspace_elements(packed), device="cuda")
        out = risa.int8_attention_from_prequantized(packed, _block_mass=workspace)
        return out, workspace

    (out_c, ws_c), (out_d, ws_d) = _both(capture)
    assert torch.equal(out_c, out_d)
    assert torch.equal(ws_c.view(torch.int32), ws_d.view(torch.int32))
