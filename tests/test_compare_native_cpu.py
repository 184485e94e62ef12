"""Host logic of the two-library comparison tool (no GPU: nothing is launched)."""
import argparse

import pytest

from risaattention_b200 import _backend, compare_native


def test_case_parsing_and_labels():
    shape = compare_native.parse_case("1,16,4,512,640,128")
    assert shape == {"batch": 1, "q_heads": 16, "kv_heads": 4, "q_len": 512, "k_len": 640,
                     "head_dim": 128}
    assert compare_native.case_label(shape) == "B1_Hq16_Hkv4_Lq512_Lk640_D128"
    for bad in ("1,16,4,512,512", "1,16,4,512,512,x", "1,16,5,512,512,128", "0,1,1,1,1,64"):
        with pytest.raises(argparse.ArgumentTypeError):
            compare_native.parse_case(bad)


def test_measurement_positions_are_mirrored():
    orders = compare_native.balanced_orders(["a", "b", "c"], 4)
    assert orders == [["a", "b", "c"], ["c", "b", "a"], ["a", "b", "c"], ["c", "b", "a"]]
    for name in "abc":  # every method is first as often as it is last
        assert sum(o[0] == name for o in orders) == sum(o[-1] == name for o in orders)


def test_calls_are_routed_and_the_module_is_restored():
    original = _backend._C
    marker = object()
    assert compare_native.with_native(marker, lambda: _backend._C) is marker
    assert _backend._C is original
    with pytest.raises(KeyError):
        compare_native.with_native(marker, lambda: {}["missing"])
    assert _backend._C is original


@pytest.mark.skipif(_backend._ABI is None, reason="library not built")
def test_a_second_copy_of_the_library_loads(tmp_path):
    import shutil

    copy = tmp_path / "librisa_b200.so"
    shutil.copy(_backend._LIB_PATH, copy)
    other = compare_native.load_library(copy)
    assert other.lib._name == str(copy) and other.lib._handle != _backend._ABI.lib._handle
    for name in ("risa_sdpa_quantize", "risa_sdpa_prequantized", "risa_dense_attention",
                 "risa_sdpa_select", "select_retained_mass_csr", "prepare_key_mask_tiles"):
        assert callable(getattr(other, name))
    with pytest.raises(FileNotFoundError):
        compare_native.load_library(tmp_path / "absent.so")


def test_arguments():
    parser = compare_native.build_parser()
    args = parser.parse_args(["--baseline-library", "x.so", "--case", "1,2,1,64,64,64", "--seed",
                              "3", "--include-components"])
    assert args.case[0]["q_heads"] == 2 and args.seed == [3] and args.include_components
    assert (args.samples, args.calls, args.warmup) == (24, 20, 20)
    with pytest.raises(SystemExit):
        parser.parse_args([])
