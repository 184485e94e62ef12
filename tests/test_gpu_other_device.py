"""Tensors on a GPU other than the thread's current one are served on their own GPU, through both
native surfaces: the library launches on the current device, so every entry point makes the device
of its tensors current for the call.  Needs two GPUs in the process; skipped otherwise."""
import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]

import risaattention_b200 as risa  # noqa: E402
from risaattention_b200 import _backend, compare_native  # noqa: E402


def _inputs(device):
    g = torch.Generator(device=device).manual_seed(31)
    q = torch.randn(1, 4, 300, 128, device=device, generator=g).bfloat16()
    k = torch.randn(1, 2, 1300, 128, device=device, generator=g).bfloat16()
    v = torch.randn(1, 2, 1300, 128, device=device, generator=g).bfloat16()
    return q, k, v


@pytest.mark.parametrize("surface", ["module", "ctypes"])
def test_calls_follow_their_tensors(surface):
    assert torch.cuda.current_device() == 0
    native = _backend._C if surface == "module" else _backend._ABI

    def every_route(device):
        q, k, v = _inputs(device)
        mask = torch.ones(1, 1, 1, 1300, dtype=torch.bool, device=device)
        mask[..., :300] = False
        dense = risa.int8_attention(q, k, v, v_quantization="midpoint_affine")
        out, lse = risa.int8_attention(q, k, v, return_lse=True, is_causal=True)
        masked = risa.int8_attention(q, k, v, attn_mask=mask)
        built, pattern = risa.construct_sparse_int8_attention(q, k, v, theta=0.9)
        sparse = risa.sparse_int8_attention(q, k, v, pattern)
        torch.cuda.synchronize(device)
        return [dense, out, lse, masked, built, sparse, pattern.row_offsets, pattern.block_indices]

    def run():
        here = every_route("cuda:0")
        there = every_route("cuda:1")  # the current device stays cuda:0
        assert torch.cuda.current_device() == 0
        for a, b in zip(here, there):
            assert b.device == torch.device("cuda:1")
            assert torch.equal(a.cpu(), b.cpu())
        with torch.cuda.device(1):
            native.device_status()
        native.device_status()

    compare_native.with_native(native, run)
