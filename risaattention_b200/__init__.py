"""B200-native RISA quantised attention: the reference package's public names
(src/risa_attention/__init__.py:17-31) over hand-written sm_100a kernels."""
from ._backend import is_available as int8_attention_is_available
from .attention import (PrequantizedInt8Attention, RetainedMassPattern,
                        build_retained_mass_pattern, construct_sparse_int8_attention,
                        construct_sparse_int8_attention_from_prequantized, int8_attention,
                        int8_attention_from_prequantized, is_available, measure_pattern_recall,
                        prequantize_int8_attention, sparse_int8_attention)
from .host_pipeline import int8_attention_from_host
from .permutation import KVPermutation, prepare_kv_permutation

__all__ = [
    "KVPermutation", "prepare_kv_permutation", "PrequantizedInt8Attention", "RetainedMassPattern",
    "build_retained_mass_pattern", "construct_sparse_int8_attention",
    "construct_sparse_int8_attention_from_prequantized", "int8_attention",
    "int8_attention_from_host", "int8_attention_from_prequantized", "int8_attention_is_available", "measure_pattern_recall",
    "prequantize_int8_attention", "sparse_int8_attention",
]
__version__ = "0.1.0"
