"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, the
Python API keeps the reference's names and error contracts, and nothing computes without a GPU."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "risa_b200.h").read_text()
    declared = set(re.findall(r"\b(risa_b200_\w+)\s*\(", header))
    assert len(declared) >= 12
    lib = ctypes.CDLL(str(ROOT / "risaattention_b200" / "librisa_b200.so"))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/risa_b200.h but not exported"
    lib.risa_b200_abi_version.restype = ctypes.c_int
    assert lib.risa_b200_abi_version() == 1


def test_contract_violations_are_reported_not_computed():
    lib = ctypes.CDLL(str(ROOT / "risaattention_b200" / "librisa_b200.so"))
    lib.risa_b200_last_error.restype = ctypes.c_char_p
    # null tensors / bad head_dim are rejected before any CUDA call
    lib.risa_b200_quantize_v_workspace_size.restype = ctypes.c_size_t
    assert lib.risa_b200_quantize_v_workspace_size(1, 4, 32768, 128) > 0
    assert lib.risa_b200_quantize_v_workspace_size(0, 4, 32768, 128) == 0
    # the combined quantiser checks V's contract first and Q/K's before any launch: null tensors are
    # a contract violation (status 1) with a message, not a crash
    c_vp, c_i32, c_i64, c_sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    lib.risa_b200_quantize_qkv.restype = c_i32
    lib.risa_b200_quantize_qkv.argtypes = ([c_vp] * 10 + [c_i32] * 8 + [c_i64] * 9 + [c_i32] * 2
                                          + [c_vp] * 4 + [c_sz, c_vp])
    status = lib.risa_b200_quantize_qkv(*([None] * 10), 1, 16, 128, 4, 128, 128, 64, 128,
                                        *([128] * 9), 2, 0, None, None, None, None, 0, None)
    assert status == 1 and b"null tensor" in lib.risa_b200_last_error()
    # scratch sizes are zero for shapes that are never split and for nonsense
    lib.risa_b200_attention_scratch_size.restype = c_sz
    assert lib.risa_b200_attention_scratch_size(0, 16, 128, 128, 128, 64) == 0
    assert lib.risa_b200_attention_scratch_size(1, 16, 128, 128, 128, 96) == 0


def test_public_names_match_reference():
    import risaattention_b200 as risa

    for name in ["KVPermutation", "prepare_kv_permutation", "PrequantizedInt8Attention",
                 "RetainedMassPattern", "build_retained_mass_pattern",
                 "construct_sparse_int8_attention",
                 "construct_sparse_int8_attention_from_prequantized", "int8_attention",
                 "int8_attention_from_prequantized", "int8_attention_is_available",
                 "measure_pattern_recall", "prequantize_int8_attention", "sparse_int8_attention"]:
        assert hasattr(risa, name)
    assert sorted(risa.__all__) == sorted(n for n in risa.__all__)
    fields = [f for f in risa.PrequantizedInt8Attention.__dataclass_fields__]
    assert fields == ["q", "k", "v", "q_scale", "k_scale", "v_scale", "v_center",
                      "original_head_dim", "input_dtype", "attention_scale", "cta_k", "attn_mask",
                      "v_quantization", "is_causal", "lse_shift", "kv_permuted"]


def test_no_cpu_fallback():
    import risaattention_b200 as risa

    assert not risa.int8_attention_is_available("cpu")
    x = torch.zeros(1, 2, 4, 64)
    with pytest.raises(ValueError, match="CUDA device"):
        risa.int8_attention(x, x, x)
    with pytest.raises(ValueError, match="shape"):
        risa.int8_attention(x[0], x, x)
    with pytest.raises(TypeError, match="float32, float16, or bfloat16"):
        risa.int8_attention(x.double(), x.double(), x.double())


def test_validation_helpers():
    from risaattention_b200._validation import (apply_score_mask, pad_key_length,
                                                select_key_block_size, uses_centered_values)

    assert select_key_block_size(128, 1025, has_mask=False) == 128
    assert select_key_block_size(128, 1024, has_mask=False) == 64
    assert select_key_block_size(64, 4096, has_mask=False) == 64
    assert select_key_block_size(256, 4096, has_mask=True) == 64
    assert pad_key_length(1025, 128) == 1152
    with pytest.raises(ValueError, match="v_quantization"):
        uses_centered_values("fp8")
    s = torch.zeros(1, 1, 3, 4)
    m = apply_score_mask(s, None, True, 0)
    assert torch.isneginf(m[0, 0, 0, 1:]).all() and m[0, 0, 2, 2] == 0


def test_pattern_properties():
    import risaattention_b200 as risa

    p = risa.RetainedMassPattern(
        row_offsets=torch.tensor([0, 2, 3], dtype=torch.int32),
        block_indices=torch.tensor([0, 3, 1], dtype=torch.int32), batch_size=1, q_heads=1,
        q_length=256, kv_length=512, query_block_size=128, key_block_size=128,
        attention_scale=0.1, retained_mass_target=0.9, measured_retained_mass=0.95)
    assert p.coverage == 3 / 8 and p.sparsity == 5 / 8 and p.index_bytes == 24


def test_fake_tensor_and_operator_schema():
    """Under fake tensors (what torch.compile traces with) the public call resolves to the
    registered ``risa_attention::*`` operators, whose shape-only implementations answer without a
    device (reference tests/contracts/test_risa_attention.py:45-52)."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import risaattention_b200 as risa
    from risaattention_b200 import dense

    assert dense.OPERATORS_REGISTERED == (True, True)
    schema = str(torch.ops.risa_attention.int8_attention.default._schema)
    assert schema == ("risa_attention::int8_attention(Tensor q, Tensor k, Tensor v, float? scale, "
                      "bool use_midpoint_affine, bool is_causal) -> Tensor")
    schema = str(torch.ops.risa_attention.int8_attention_masked.default._schema)
    assert schema == ("risa_attention::int8_attention_masked(Tensor q, Tensor k, Tensor v, "
                      "Tensor attn_mask, float? scale, bool use_midpoint_affine, bool is_causal) "
                      "-> Tensor")
    with FakeTensorMode():
        q = torch.empty(1, 2, 17, 64, device="cuda")
        for mode in ("midpoint_affine", "absmax"):
            out = risa.int8_attention(q, q, q, is_causal=True, v_quantization=mode)
            assert out.shape == q.shape and out.device == q.device and out.dtype == q.dtype
        mask = torch.ones(17, 17, dtype=torch.bool, device="cuda")
        assert risa.int8_attention(q, q, q, attn_mask=mask).shape == q.shape
    with pytest.raises(ValueError, match="v_quantization"):
        risa.int8_attention(torch.empty(1), torch.empty(1), torch.empty(1), v_quantization="x")


def test_split_last_wave_rule_known_answers():
    """The rule that decides whether the one-call dense path adds a merge launch is a pure function
    of the launch shape; known answers for a 148-SM GPU."""
    lib = ctypes.CDLL(str(ROOT / "risaattention_b200" / "librisa_b200.so"))
    parts = lib.risa_b200_split_last_wave_parts
    parts.restype = ctypes.c_int
    assert parts(4096, 256, 128, 148) == 4   # 16 heads at 32K: 100 CTAs -> 400 quarters = 3 rounds of 1/4
    assert parts(1280, 256, 128, 148) == 3   # 5 heads at 32K: 96 CTAs -> 288 thirds = 2 rounds of 1/3
    assert parts(2048, 256, 128, 148) == 0   # 8 heads at 32K: 124 CTAs, no cut fills the rounds better
    assert parts(512, 256, 128, 148) == 2    # 2 heads at 32K (one of 8 GPUs): 68 CTAs, 2 parts each
    assert parts(1024, 256, 128, 148) == 0   # 4 heads at 32K: 136 CTAs
    assert parts(512, 32, 128, 148) == 2     # 16 heads at 4K
    assert parts(160, 32, 128, 148) == 4     # 5 heads at 4K: 12 CTAs, 4 parts each
    assert parts(160, 16, 128, 148) == 0     # 2K: the saving would be below 2048 keys
    assert parts(128, 256, 128, 148) == 0    # less than one wave
    assert parts(296, 256, 128, 148) == 0    # whole waves only
    assert parts(512, 256, 128, 0) == 0


def test_public_call_passes_causal_flag_and_value_mode_to_the_launch():
    """Every combination of V mode, causal flag and mask presence reaches the function that
    launches the kernels unchanged (after reference tests/contracts/test_risa_attention.py:29-43)."""
    from unittest.mock import patch

    import risaattention_b200 as risa
    from risaattention_b200 import dense

    q = torch.randn(1, 2, 3, 64)
    for mode in ("midpoint_affine", "absmax"):
        for causal in (False, True):
            for mask in (None, torch.ones(3, 3, dtype=torch.bool)):
                with patch.object(dense, "execute_dense_attention",
                                  return_value=q.clone()) as launch:
                    risa.int8_attention(q, q, q, attn_mask=mask, is_causal=causal,
                                        v_quantization=mode)
                assert launch.call_count == 1
                assert launch.call_args.kwargs["is_causal"] == causal
                assert launch.call_args.kwargs["use_midpoint_affine"] == (mode == "midpoint_affine")
                assert (launch.call_args.kwargs["attn_mask"] is None) == (mask is None)


def test_mask_identity_follows_in_place_writes():
    """A retained pattern is bound to the mask it was built with: an in-place write changes the
    mask's identity; masked and causal scores follow the FP32 specification (after reference
    tests/contracts/test_risa_attention.py:59-67)."""
    from risaattention_b200._validation import apply_score_mask, mask_signature

    mask = torch.ones(1, 1, 3, 5, dtype=torch.bool)
    before = mask_signature(mask)
    assert before == mask_signature(mask)
    mask[..., 0] = False
    assert before != mask_signature(mask)
    assert mask_signature(None) is None
    scores = apply_score_mask(torch.zeros(1, 1, 3, 5), mask, True, 0)
    assert torch.isneginf(scores[..., 0, :]).all()
    assert torch.isneginf(scores[..., 1, 2:]).all()
    assert scores[0, 0, 1, 1] == 0
    bias = torch.full((1, 1, 3, 5), 0.5)
    assert torch.equal(apply_score_mask(torch.zeros(1, 1, 3, 5), bias, False, 0), bias)
