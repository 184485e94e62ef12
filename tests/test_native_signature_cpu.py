"""The native object is a drop-in for the reference's ``_C`` module only if every call the
reference's Python runtime makes binds to it.  ``tests/golden/reference_native_calls.json`` holds
the shape of each such call (extracted from the reference's sources by
tests/golden/make_native_calls.py); here each one is bound against ``_backend._Native``."""
import inspect
import json
from pathlib import Path

import pytest

from risaattention_b200 import _backend

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_native_calls.json"
CALLS = json.loads(GOLDEN.read_text())
# what the reference splats into the recorded calls: the 12-tuple of packed operands
# (_execution.py:279-292), the optional gather-table pointer (_quantization.py:141) and the
# optional key-mask tile list (_execution.py:311,321 / :105-107,129)
STAR_ARGS = {"risa_sdpa_prequantized": 12, "risa_sdpa_quantize": 1}
STAR_KWARGS = {"risa_sdpa_prequantized": ["key_mask_tiles"], "risa_sdpa": ["key_mask_tiles"]}


def test_fixture_covers_every_entry_point_of_the_reference_module():
    names = {c["entry_point"] for c in CALLS}
    assert names == {"risa_sdpa", "risa_sdpa_quantize", "risa_sdpa_prequantized",
                     "select_retained_mass_csr", "retained_mass_selector_workspace_size",
                     "prepare_key_mask_tiles", "risa_lse_shift"}
    assert _backend._Native.fused_gather_version == 1  # csrc/bindings.cpp:655


@pytest.mark.parametrize("call", CALLS, ids=lambda c: f"{c['entry_point']}@{c['line']}")
def test_reference_call_binds(call):
    method = getattr(_backend._Native, call["entry_point"])
    signature = inspect.signature(method)
    for extra_args in ([0, STAR_ARGS.get(call["entry_point"], 0)] if call["star_args"] else [0]):
        for extra_kw in ([[], STAR_KWARGS.get(call["entry_point"], [])] if call["star_kwargs"]
                         else [[]]):
            args = [object()] * (1 + call["positional"] + extra_args)  # self + positionals
            kwargs = {name: object() for name in call["keywords"] + extra_kw}
            if call["entry_point"] == "risa_sdpa_prequantized" and extra_args == 0:
                continue  # that call always splats its 12 operands
            signature.bind(*args, **kwargs)


def test_fixture_is_current():
    reference = Path("/root/reference")
    if not (reference / "src" / "risa_attention").is_dir():
        pytest.skip("reference sources not mounted")
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "make_native_calls", GOLDEN.parent / "make_native_calls.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    assert module.extract(reference) == CALLS


def test_keyword_names_and_defaults_match_the_reference_module():
    """Keyword names and defaults of the registered functions (csrc/bindings.cpp:642-673)."""
    def params(name):
        return list(inspect.signature(getattr(_backend._Native, name)).parameters.values())[1:]

    sdpa = params("risa_sdpa")
    assert [p.name for p in sdpa] == [
        "q", "k", "v", "o", "q_int8", "q_scale", "k_int8", "k_scale", "v_int8", "v_scale",
        "v_center", "sm_scale", "input_dtype_code", "output_dtype_code", "use_midpoint_affine",
        "stream_ptr", "anchor_indices_ptr", "attn_mask", "cta_k", "is_causal", "key_mask_tiles"]
    assert [p.default for p in sdpa[17:]] == [None, 0, False, None]
    quantize = params("risa_sdpa_quantize")
    assert [p.name for p in quantize[:16]] == [
        "q", "k", "v", "q_int8", "q_scale", "k_int8", "k_scale", "v_int8", "v_scale", "v_center",
        "cta_k", "input_dtype_code", "use_midpoint_affine", "stream_ptr", "anchor_indices_ptr",
        "permutation_ptr"]
    assert quantize[15].default == 0
    pre = params("risa_sdpa_prequantized")
    assert [p.name for p in pre] == [
        "q_int8", "k_int8", "v_int8", "o", "q_scale", "k_scale", "v_scale", "v_center", "cta_k",
        "sm_scale", "output_dtype_code", "stream_ptr", "attn_mask", "sparse_row_offsets",
        "sparse_block_indices", "block_mass", "is_causal", "lse", "key_mask_tiles"]
    assert [p.default for p in pre[12:]] == [None, None, None, None, False, None, None]


def _extension_parameters(name):
    """(parameter names, names that have defaults) of a function of the C++ extension, read from
    the signature line pybind11 puts at the top of its docstring."""
    line = getattr(_backend._C, name).__doc__.splitlines()[0]
    inside = line[line.index("(") + 1:line.rindex(")")]
    names, defaults, depth, token = [], set(), 0, ""
    for ch in inside + ",":
        if ch in "[(":
            depth += 1
        elif ch in "])":
            depth -= 1
        if ch == "," and depth == 0:
            token = token.strip()
            if token and token != "*":
                name_part = token.split(":")[0].strip()
                names.append(name_part)
                if "=" in token:
                    defaults.add(name_part)
            token = ""
        else:
            token += ch
    return names, defaults


@pytest.mark.parametrize("call", CALLS, ids=lambda c: f"{c['entry_point']}@{c['line']}")
def test_reference_call_fits_the_cpp_extension(call):
    """The PyTorch C++ extension takes the same calls: enough positional parameters, every keyword
    the reference uses present by name, everything the reference leaves out defaulted."""
    if _backend._C is None:
        pytest.skip(f"extension not built: {_backend._EXTENSION_ERROR}")
    names, defaults = _extension_parameters(call["entry_point"])
    reference = inspect.signature(getattr(_backend._Native, call["entry_point"]))
    reference_names = [n for n in reference.parameters if n != "self"]
    assert names == reference_names  # same order and names as the ctypes surface checked above
    positional = call["positional"] + (STAR_ARGS.get(call["entry_point"], 0)
                                       if call["star_args"] else 0)
    used = set(names[:positional]) | set(call["keywords"])
    if call["star_kwargs"]:
        assert set(STAR_KWARGS.get(call["entry_point"], [])) <= set(names)
    assert set(call["keywords"]) <= set(names)
    assert all(n in defaults for n in names if n not in used)
