"""The native module refuses buffers the kernels would index out of bounds, before any launch: the
checks (and their messages) of the reference module's entry points, csrc/bindings.cpp:52-140,
196-246 and 290-432.  Every case here fails a check, so nothing runs on a device and the tests
need no GPU."""
import pytest
import torch

from risaattention_b200 import _backend

pytestmark = pytest.mark.skipif(_backend._C is None, reason="native module not built")


def _attend_arguments(**changes):
    """A consistent set of packed operands (batch 1, 2 query heads on 1 KV head, 130 queries,
    70 keys in 64-key tiles, head_dim 64), with single arguments replaced."""
    a = {
        "q_int8": torch.zeros(1, 2, 130, 64, dtype=torch.int8),
        "k_int8": torch.zeros(1, 1, 70, 64, dtype=torch.int8),
        "v_int8": torch.zeros(64, 128, dtype=torch.int8),
        "o": torch.zeros(1, 2, 130, 64, dtype=torch.bfloat16),
        "q_scale": torch.ones(1, 2, 64),
        "k_scale": torch.ones(1, 1, 8),
        "v_scale": torch.ones(64),
        "v_center": torch.zeros(64),
        "cta_k": 64, "sm_scale": 0.125, "output_dtype_code": 2, "stream_ptr": 0,
    }
    a.update(changes)
    return a


ATTEND_CASES = [
    ({"cta_k": 96}, "cta_k must be 64 or 128"),
    ({"cta_k": 0}, "cta_k must be 64 or 128"),
    ({"output_dtype_code": 0}, "output_dtype_code must be 1"),
    ({"v_int8": torch.zeros(1, 64, 128, dtype=torch.int8)}, "packed v must be 2D"),
    ({"cta_k": 128}, "cta_k 128 requires head_dim 128 or 256"),
    ({"sparse_row_offsets": torch.zeros(5, dtype=torch.int32)}, "provided together"),
    ({"sparse_row_offsets": torch.zeros(5, dtype=torch.int32),
      "sparse_block_indices": torch.zeros(4, dtype=torch.int32),
      "block_mass": torch.zeros(8 + 2 * 130 * 6)}, "block mass requires dense attention"),
    ({"v_int8": torch.zeros(64, 64, dtype=torch.int8)}, "incompatible quantized tensor shapes"),
    ({"o": torch.zeros(1, 2, 130, 64)}, "packed operands must be int8"),
    ({"q_int8": torch.zeros(1, 2, 130, 64, dtype=torch.uint8)}, "packed operands must be int8"),
    ({"q_scale": torch.ones(1, 2, 32)}, "scale and centre tensors"),
    ({"k_scale": torch.ones(1, 1, 4)}, "scale and centre tensors"),
    ({"v_center": torch.zeros(32)}, "scale and centre tensors"),
    ({"q_int8": torch.zeros(1, 2, 64, 130, dtype=torch.int8).transpose(2, 3)},
     "quantized tensors must be contiguous"),
    ({"lse": torch.zeros(1, 2, 129)}, "LSE must be contiguous float32"),
    ({"attn_mask": torch.ones(1, 2, 130, 71, dtype=torch.bool)}, "attention mask must be expanded"),
    ({"attn_mask": torch.ones(1, 2, 130, 70, dtype=torch.int32)},
     "attention mask must be bool, float16, bfloat16, or float32"),
    ({"sparse_row_offsets": torch.zeros(4, dtype=torch.int32),
      "sparse_block_indices": torch.zeros(4, dtype=torch.int32)}, "sparse support must be"),
    ({"sparse_row_offsets": torch.zeros(5, dtype=torch.int64),
      "sparse_block_indices": torch.zeros(4, dtype=torch.int32)}, "sparse support must be"),
    ({"sparse_row_offsets": torch.zeros(5, dtype=torch.int32),
      "sparse_block_indices": torch.zeros(0, dtype=torch.int32)}, "non-empty and contiguous"),
    ({"sparse_row_offsets": torch.zeros(5, dtype=torch.int32),
      "sparse_block_indices": torch.zeros(8, dtype=torch.int32)[::2]}, "non-empty and contiguous"),
    ({"block_mass": torch.zeros(8 + 2 * 130 * 6 - 1)}, "block_mass workspace must contain"),
    ({"block_mass": torch.zeros(8 + 2 * 130 * 6, dtype=torch.float64)},
     "block_mass workspace must contain"),
    # on the host, and with the wrong width
    ({"key_mask_tiles": torch.zeros(1, 2, 3, dtype=torch.int32)}, "key mask tiles must be"),
]


@pytest.mark.parametrize("changes,message", ATTEND_CASES)
def test_attention_entry_refuses_inconsistent_buffers(changes, message):
    with pytest.raises(RuntimeError, match=message):
        _backend._C.risa_sdpa_prequantized(**_attend_arguments(**changes))


def _quantize_arguments(**changes):
    a = {
        "q": torch.zeros(1, 2, 130, 64, dtype=torch.bfloat16),
        "k": torch.zeros(1, 1, 70, 64, dtype=torch.bfloat16),
        "v": torch.zeros(1, 1, 70, 64, dtype=torch.bfloat16),
        "q_int8": torch.zeros(1, 2, 130, 64, dtype=torch.int8),
        "q_scale": torch.ones(1, 2, 64),
        "k_int8": torch.zeros(1, 1, 70, 64, dtype=torch.int8),
        "k_scale": torch.ones(1, 1, 8),
        "v_int8": torch.zeros(64, 128, dtype=torch.int8),
        "v_scale": torch.ones(64),
        "v_center": torch.zeros(64),
        "cta_k": 64, "input_dtype_code": 2, "use_midpoint_affine": False, "stream_ptr": 0,
        "anchor_indices_ptr": torch.zeros(1, dtype=torch.int32),
    }
    a.update(changes)
    return a


QUANTIZE_CASES = [
    ({"v": torch.zeros(1, 70, 64, dtype=torch.bfloat16)}, "q, k, and v must be 4D"),
    ({"cta_k": 32}, "cta_k must be 64 or 128"),
    ({"input_dtype_code": 3}, "input_dtype_code must be 0"),
    ({"anchor_indices_ptr": 0}, "anchor_indices scratch is required"),
    ({"anchor_indices_ptr": None}, "anchor_indices scratch is required"),
    ({"v": torch.zeros(1, 1, 71, 64, dtype=torch.bfloat16)}, "incompatible q, k, and v shapes"),
    ({"k": torch.zeros(1, 1, 70, 128, dtype=torch.bfloat16)}, "incompatible q, k, and v shapes"),
    ({"input_dtype_code": 1}, "must have the element type"),
    ({"q_int8": torch.zeros(1, 2, 128, 64, dtype=torch.int8)}, "incompatible INT8 output shapes"),
    ({"v_int8": torch.zeros(64, 70, dtype=torch.int8)}, "incompatible INT8 output shapes"),
    ({"k_int8": torch.zeros(1, 1, 70, 64, dtype=torch.uint8)}, "incompatible INT8 output shapes"),
    ({"q_scale": torch.ones(1, 2, 63)}, "scale and centre tensors"),
    ({"v_scale": torch.ones(128)[::2]}, "scale and centre tensors"),
]


@pytest.mark.parametrize("changes,message", QUANTIZE_CASES)
def test_quantize_entry_refuses_inconsistent_buffers(changes, message):
    with pytest.raises(RuntimeError, match=message):
        _backend._C.risa_sdpa_quantize(**_quantize_arguments(**changes))


def _selector_arguments(rows=3, tiles=5, **changes):
    a = {
        "sorted_mass": torch.zeros(rows, tiles),
        "descending_indices": torch.zeros(rows, tiles, dtype=torch.int64),
        "counts": torch.zeros(rows, dtype=torch.int32),
        "support": torch.zeros(rows, tiles, dtype=torch.uint8),
        "row_totals": torch.zeros(rows, 2, dtype=torch.float64),
        "row_offsets": torch.zeros(rows + 1, dtype=torch.int32),
        "block_indices": torch.zeros(rows * tiles, dtype=torch.int32),
        "summary": torch.zeros(3, dtype=torch.float64),
        "scan_workspace": torch.zeros(
            _backend._C.retained_mass_selector_workspace_size(rows), dtype=torch.uint8),
        "theta": 0.9, "stream_ptr": 0,
    }
    a.update(changes)
    return a


SELECTOR_CASES = [
    ({"sorted_mass": torch.zeros(15)}, "masses and indices must be 2D"),
    ({"sorted_mass": torch.zeros(0, 5), "descending_indices": torch.zeros(0, 5, dtype=torch.int64)},
     "invalid shape, dtype, or stride"),
    ({"sorted_mass": torch.zeros(3, 5, dtype=torch.float64)}, "invalid shape, dtype, or stride"),
    ({"descending_indices": torch.zeros(3, 5, dtype=torch.int32)}, "invalid shape, dtype, or stride"),
    ({"counts": torch.zeros(4, dtype=torch.int32)}, "invalid shape, dtype, or stride"),
    ({"support": torch.zeros(3, 5, dtype=torch.bool)}, "invalid shape, dtype, or stride"),
    ({"row_totals": torch.zeros(3, 2)}, "invalid shape, dtype, or stride"),
    ({"row_offsets": torch.zeros(3, dtype=torch.int32)}, "invalid shape, dtype, or stride"),
    ({"block_indices": torch.zeros(14, dtype=torch.int32)}, "invalid shape, dtype, or stride"),
    ({"summary": torch.zeros(2, dtype=torch.float64)}, "invalid shape, dtype, or stride"),
    ({"sorted_mass": torch.zeros(5, 3).t()}, "invalid shape, dtype, or stride"),
    ({"scan_workspace": torch.zeros(0, dtype=torch.uint8)}, "scan workspace is too small"),
]


@pytest.mark.parametrize("changes,message", SELECTOR_CASES)
def test_selector_entry_refuses_inconsistent_buffers(changes, message):
    if _backend._C.retained_mass_selector_workspace_size(3) == 0 and "too small" in message:
        pytest.skip("the selector needs no scan workspace for so few rows")
    with pytest.raises(RuntimeError, match=message):
        _backend._C.select_retained_mass_csr(**_selector_arguments(**changes))


def test_key_mask_tile_entry_refuses_inconsistent_buffers():
    broadcast = torch.ones(1, 1, 1, 200, dtype=torch.bool).expand(1, 2, 130, 200)
    tiles = torch.zeros(1, 2, 5, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="expanded broadcast key mask"):
        _backend._C.prepare_key_mask_tiles(torch.ones(1, 2, 130, 200, dtype=torch.bool), tiles, 64, 0)
    with pytest.raises(RuntimeError, match="expanded broadcast key mask"):
        _backend._C.prepare_key_mask_tiles(broadcast, tiles, 32, 0)
    # tile list on the host / of the wrong width
    with pytest.raises(RuntimeError, match="key mask tiles must be contiguous CUDA int32"):
        _backend._C.prepare_key_mask_tiles(broadcast, tiles, 64, 0)
    with pytest.raises(RuntimeError, match="key mask tiles must be contiguous CUDA int32"):
        _backend._C.prepare_key_mask_tiles(broadcast, torch.zeros(1, 2, 4, dtype=torch.int32), 64, 0)


@pytest.mark.parametrize("shape", [(1, 4, 2, 300, 1300, 128, 128), (2, 2, 2, 130, 70, 64, 64),
                                   (1, 2, 1, 128, 1025, 256, 64)])
def test_one_call_allocation_matches_the_python_allocations(shape):
    """The module's single allocation call hands out the same nine buffers (shape, element type)
    as the allocations the Python layer falls back to on a surface without it."""
    from risaattention_b200._quantization import PackedBuffers

    batch, q_heads, kv_heads, q_len, k_len, dim, tile = shape
    q = torch.zeros(batch, q_heads, q_len, dim)
    k = torch.zeros(batch, kv_heads, k_len, dim)
    names = ("q_codes", "k_codes", "q_scales", "k_scales", "v_codes", "v_scales", "v_centers",
             "anchors", "workspace")
    through_module = PackedBuffers(q, k, tile)
    original = _backend._C

    class WithoutAllocation:
        def __getattr__(self, name):
            if name == "allocate_packed":
                raise AttributeError(name)
            return getattr(original, name)

    _backend._C = WithoutAllocation()
    try:
        from_python = PackedBuffers(q, k, tile)
    finally:
        _backend._C = original
    assert through_module.padded_key_length == from_python.padded_key_length
    for name in names:
        a, b = getattr(through_module, name), getattr(from_python, name)
        assert a.shape == b.shape and a.dtype == b.dtype and a.is_contiguous(), name
