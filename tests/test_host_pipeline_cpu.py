"""Argument contract of the host-operand entry point (everything that is decided before a CUDA
call is made)."""
import pytest
import torch

import risaattention_b200 as risa


def _qkv():
    q = torch.zeros(1, 4, 16, 128, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 32, 128, dtype=torch.bfloat16)
    return q, k, k.clone()


@pytest.mark.parametrize("kwargs", [{"return_lse": True}, {"attn_mask": torch.ones(16, 32)},
                                    {"kv_permutation": object()}])
def test_unsupported_options_are_refused(kwargs):
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="does not support"):
        risa.int8_attention_from_host(q, k, v, **kwargs)


def test_shape_and_head_contract():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="expected q"):
        risa.int8_attention_from_host(q[0], k, v)
    with pytest.raises(ValueError, match="expected q"):
        risa.int8_attention_from_host(q, k, v[:, :1])
    with pytest.raises(ValueError, match="divisible"):
        risa.int8_attention_from_host(torch.zeros(1, 3, 16, 128), torch.zeros(1, 2, 32, 128),
                                      torch.zeros(1, 2, 32, 128))
