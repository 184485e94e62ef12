"""The allocation-free V quantiser (risa_b200_quantize_v_static) against the ordinary entry point.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.  Some callers of the library cannot allocate device memory when they call it -- a
server that froze its memory budget at start-up, or a cgo / JNI / ctypes host with no device
allocator -- so this entry point keeps its scratch in a fixed array inside the library.  The test
calls it through the C-ABI twice in a row on different data (the array keeps the first call's
contents, which must not leak into the second) and requires bit-identical results to
risa_b200_quantize_v, then checks that an oversized problem is refused."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, name, v, padded, affine, workspace=None):
    b, h, n, d = v.shape
    codes = torch.empty(b * h * d, padded, dtype=torch.int8, device=v.device)
    scale = torch.empty(b * h * d, device=v.device)
    center = torch.empty(b * h * d, device=v.device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    args = [p(v), p(codes), p(scale), p(center), b, h, n, d, padded, v.stride(0), v.stride(1),
            v.stride(2), 2, int(affine), None]
    if workspace is not None:
        args += [p(workspace), workspace.numel()]
    args.append(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    status = getattr(lib, name)(*args)
    torch.cuda.synchronize()
    return status, codes, scale, center


def test_static_scratch_matches_workspace_entry_point():
    from risaattention_b200 import _backend

    lib = _backend._ABI.lib
    limit = lib.risa_b200_quantize_v_static_limit()
    assert limit == 4 << 20
    g = torch.Generator(device="cuda").manual_seed(123)
    for call, (heads, length) in enumerate([(4, 4097), (2, 1500)]):  # two calls in a row
        v = (torch.randn(1, heads, length, 128, device="cuda", generator=g) + call).bfloat16()
        padded = -(-length // 128) * 128
        need = lib.risa_b200_quantize_v_workspace_size(1, heads, length, 128)
        assert 0 < need <= limit
        workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        for affine in (False, True):
            s0, c0, sc0, ce0 = _call(lib, "risa_b200_quantize_v", v, padded, affine, workspace)
            s1, c1, sc1, ce1 = _call(lib, "risa_b200_quantize_v_static", v, padded, affine)
            assert s0 == 0 and s1 == 0, lib.risa_b200_last_error().decode()
            assert torch.equal(c0, c1) and torch.equal(sc0, sc1) and torch.equal(ce0, ce1)


def test_static_scratch_rejects_oversized_problem():
    from risaattention_b200 import _backend

    lib = _backend._ABI.lib
    heads, length = 40, 32768                       # needs ~13 MiB of scratch
    assert lib.risa_b200_quantize_v_workspace_size(1, heads, length, 128) > \
        lib.risa_b200_quantize_v_static_limit()
    v = torch.zeros(1, 1, 16, 128, device="cuda", dtype=torch.bfloat16)  # never read
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    status = lib.risa_b200_quantize_v_static(p(v), p(v), p(v), p(v), 1, heads, length, 128, length,
                                             0, 0, 128, 2, 0, None, None)
    assert status == 1
    assert b"scratch" in lib.risa_b200_last_error()
