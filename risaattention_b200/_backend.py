"""The native module the runtime calls, and a ctypes view of the C-ABI beneath it.

The reference binds its kernels through a nanobind module ``_C`` that receives DLPack capsules
(src/risa_attention/_backend.py:6-54, csrc/bindings.cpp:642-673).  Here ``_C`` is the PyTorch C++
extension built from csrc/torch_binding.cpp: the same entry-point names, argument order, keyword
names and defaults over the C-ABI library ``librisa_b200.so`` (include/risa_b200.h), so the
reference's own Python runtime can call it unchanged: tensor arguments may be ``torch.Tensor``
objects or DLPack capsules, scratch pointers (``anchor_indices_ptr``, ``permutation_ptr``) may be
tensors or raw integer addresses, the stream is the raw ``cudaStream_t``.

``_Native`` is the same surface written against the shared library with ctypes alone, for hosts
that have no C++ toolchain or no torch headers at build time and for tests that drive the C-ABI
symbol by symbol (``_ABI.lib``); it calls exactly the same library functions.

There is no CPU fallback: when the extension or a capable GPU is missing every entry point raises
``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import functools
from pathlib import Path

import torch

REQUIRED_COMPUTE_CAPABILITY_MAJOR = 10  # the library holds sm_100a code only
_LIB_PATH = Path(__file__).resolve().parent / "librisa_b200.so"
_EXTENSION_ERROR: Exception | None = None

c_i32, c_i64, c_f32, c_f64, c_vp, c_sz = (
    ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t,
)

_SIGNATURES = {
    "risa_b200_last_error": (ctypes.c_char_p, []),
    "risa_b200_abi_version": (c_i32, []),
    "risa_b200_quantize_qk": (c_i32, [c_vp] * 6 + [c_i32] * 7 + [c_i64] * 6 + [c_i32] + [c_vp] * 4),
    "risa_b200_quantize_qkv": (
        c_i32, [c_vp] * 10 + [c_i32] * 8 + [c_i64] * 9 + [c_i32] * 2 + [c_vp] * 4 + [c_sz, c_vp]),
    "risa_b200_split_last_wave_parts": (c_i32, [c_i32] * 4),
    "risa_b200_quantize_v_workspace_size": (c_sz, [c_i32] * 4),
    "risa_b200_quantize_v": (
        c_i32, [c_vp] * 4 + [c_i32] * 5 + [c_i64] * 3 + [c_i32] * 2 + [c_vp, c_vp, c_sz, c_vp]),
    "risa_b200_quantize_v_static_limit": (c_sz, []),
    "risa_b200_quantize_v_static": (
        c_i32, [c_vp] * 4 + [c_i32] * 5 + [c_i64] * 3 + [c_i32] * 2 + [c_vp, c_vp]),
    "risa_b200_attention": (
        c_i32,
        [c_vp] * 9 + [c_i64] * 4 + [c_i32] * 8 + [c_i64] * 3 + [c_f32, c_i32, c_vp, c_vp, c_vp,
                                                                   c_i32, c_vp, c_vp, c_vp]),
    "risa_b200_attention_scratch_size": (c_sz, [c_i32] * 6),
    "risa_b200_attention_scratch": (
        c_i32,
        [c_vp] * 9 + [c_i64] * 4 + [c_i32] * 8 + [c_i64] * 3 + [c_f32, c_i32, c_vp, c_vp, c_vp,
                                                                   c_i32, c_vp, c_vp, c_vp, c_sz,
                                                                   c_vp]),
    "risa_b200_select_scratch_size": (c_sz, [c_i32] * 2),
    "risa_b200_select_max_key_tiles": (c_i32, [c_i32]),
    "risa_b200_attention_select": (
        c_i32,
        [c_vp] * 9 + [c_i64] * 4 + [c_i32] * 8 + [c_i64] * 3 + [c_f32, c_i32, c_i32, c_f64, c_vp,
                                                                   c_sz, c_vp, c_vp, c_vp, c_vp,
                                                                   c_vp]),
    "risa_b200_pack_selected": (c_i32, [c_vp] * 6 + [c_i32, c_i32, c_vp]),
    "risa_b200_dense_scratch_size": (c_sz, [c_i32] * 7),
    "risa_b200_dense_attention": (
        c_i32, [c_vp] * 5 + [c_sz] + [c_i32] * 7 + [c_i64] * 9 + [c_i32, c_i32, c_f32, c_i32] +
        [c_i64] * 3 + [c_i32, c_vp]),
    "risa_b200_bounded_wait_self_test": (c_i32, [ctypes.c_uint64, c_vp]),
    "risa_b200_set_attention_path": (c_i32, [c_i32]),
    "risa_b200_device_status": (c_i32, []),
    "risa_b200_selector_workspace_size": (c_sz, [c_i32]),
    "risa_b200_select_retained_mass": (
        c_i32, [c_vp] * 9 + [c_sz, c_i32, c_i32, c_f64, c_vp]),
    "risa_b200_prepare_key_mask_tiles": (c_i32, [c_vp, c_vp] + [c_i32] * 4 + [c_i64] * 3 + [c_i32, c_vp]),
    "risa_b200_correct_lse": (
        c_i32, [c_vp] * 4 + [c_i32] * 5 + [c_i64] * 6 + [c_f32, c_i32, c_vp]),
}

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.bool: 3}


def _t(x):
    """Tensor view of a native-call argument: tensors pass through, DLPack capsules (what the
    reference's runtime hands to its native module) are imported without a copy."""
    if x is None or isinstance(x, torch.Tensor):
        return x
    return torch.utils.dlpack.from_dlpack(x)


def _ptr(x):
    """Device address of a tensor, or a raw integer address (0 / None = null)."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x) if x else None
    return ctypes.c_void_p(x.data_ptr())


def _on_device_of_first_tensor(method):
    """The library launches on the thread's current device: make the device of the call's first
    tensor current for the duration of the call, so that tensors on another GPU are served there
    (the C++ module does the same with a device guard)."""

    @functools.wraps(method)
    def call(self, first, *args, **kwargs):
        first = _t(first)
        if not first.is_cuda:
            return method(self, first, *args, **kwargs)
        with torch.cuda.device(first.device):
            return method(self, first, *args, **kwargs)

    return call


def _default_cta_k(head_dim, key_length, has_mask):
    # csrc/bindings.cpp:549-551
    return 128 if (not has_mask and head_dim >= 128 and key_length > 1024) else 64


class _Native:
    """ctypes view of librisa_b200.so with the reference's native entry-point names."""

    fused_gather_version = 1

    def __init__(self, path: Path):
        self.lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = restype, argtypes

    def _check(self, status: int):
        if status != 0:
            raise RuntimeError(self.lib.risa_b200_last_error().decode())

    # -- risa_sdpa_quantize (csrc/bindings.cpp:195-272) ---------------------------------------
    @_on_device_of_first_tensor
    def risa_sdpa_quantize(self, q, k, v, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale,
                           v_center, cta_k, input_dtype_code, use_midpoint_affine, stream_ptr,
                           anchor_indices_ptr, permutation_ptr=0, *, q_permutation_ptr=0,
                           workspace=None):
        """``permutation_ptr``: int32 [B,Hkv,Lk] gather table applied to K and V (the reference's
        fused gather); ``q_permutation_ptr`` (extension) the same for Q.  ``workspace``
        (extension): scratch for the V quantiser; allocated on the call's stream when omitted."""
        q, k, v, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale, v_center = map(
            _t, (q, k, v, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale, v_center))
        b, hq, lq, d = q.shape
        hkv, lk = k.shape[1], k.shape[2]
        if workspace is None:
            with torch.cuda.device(q.device), torch.cuda.stream(
                    torch.cuda.ExternalStream(stream_ptr, device=q.device) if stream_ptr
                    else torch.cuda.default_stream(q.device)):
                workspace = torch.empty(self.quantize_v_workspace_size(b, hkv, lk, d),
                                        dtype=torch.uint8, device=q.device)
        self._check(self.lib.risa_b200_quantize_qkv(
            _ptr(q), _ptr(q_int8), _ptr(q_scale), _ptr(k), _ptr(k_int8), _ptr(k_scale), _ptr(v),
            _ptr(v_int8), _ptr(v_scale), _ptr(v_center), b, hq, lq, hkv, lk, d, cta_k,
            v_int8.shape[1], q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1),
            k.stride(2), v.stride(0), v.stride(1), v.stride(2), input_dtype_code,
            int(use_midpoint_affine), _ptr(anchor_indices_ptr), _ptr(q_permutation_ptr),
            _ptr(permutation_ptr), _ptr(workspace), workspace.numel() * workspace.element_size(),
            stream_ptr))

    # -- risa_sdpa (csrc/bindings.cpp:497-616) ----------------------------------------------------
    @_on_device_of_first_tensor
    def risa_sdpa(self, q, k, v, o, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale, v_center,
                  sm_scale, input_dtype_code, output_dtype_code, use_midpoint_affine, stream_ptr,
                  anchor_indices_ptr, attn_mask=None, cta_k=0, is_causal=False,
                  key_mask_tiles=None):
        """Quantise Q, K and V into the caller's packed buffers and attend, on one stream."""
        # a DLPack capsule can be imported once: resolve every operand here, before the two stages
        (q, k, v, o, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale, v_center, attn_mask,
         key_mask_tiles) = map(_t, (q, k, v, o, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale,
                                    v_center, attn_mask, key_mask_tiles))
        if q.ndim != 4 or k.ndim != 4 or v.ndim != 4 or o.ndim != 4:
            raise RuntimeError("risa_sdpa: q, k, v, o must be 4D [batch_size,num_heads,L,head_dim]")
        if not 0 <= input_dtype_code <= 2:
            raise RuntimeError(
                "risa_sdpa: input_dtype_code must be 0 (fp32), 1 (fp16), or 2 (bf16)")
        if not anchor_indices_ptr and not isinstance(anchor_indices_ptr, torch.Tensor):
            raise RuntimeError("risa_sdpa: anchor_indices scratch is required")
        if cta_k == 0:
            cta_k = _default_cta_k(q.shape[3], k.shape[2], attn_mask is not None)
        self.risa_sdpa_quantize(q, k, v, q_int8, q_scale, k_int8, k_scale, v_int8, v_scale,
                                v_center, cta_k, input_dtype_code, use_midpoint_affine,
                                stream_ptr, anchor_indices_ptr)
        self.risa_sdpa_prequantized(q_int8, k_int8, v_int8, o, q_scale, k_scale, v_scale,
                                    v_center, cta_k, sm_scale, output_dtype_code, stream_ptr,
                                    attn_mask=attn_mask, is_causal=is_causal,
                                    key_mask_tiles=key_mask_tiles)

    # -- fused unmasked dense call (no counterpart in the reference's native module) ------------
    def dense_scratch_size(self, batch, q_heads, q_len, kv_heads, k_len, head_dim, cta_k) -> int:
        return int(self.lib.risa_b200_dense_scratch_size(batch, q_heads, q_len, kv_heads, k_len,
                                                         head_dim, cta_k))

    @_on_device_of_first_tensor
    def risa_dense_attention(self, q, k, v, o, scratch, cta_k, input_dtype_code,
                             use_midpoint_affine, sm_scale, output_dtype_code, is_causal,
                             stream_ptr):
        b, hq, lq, d = q.shape
        hkv, lk = k.shape[1], k.shape[2]
        self._check(self.lib.risa_b200_dense_attention(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), scratch.data_ptr(),
            scratch.numel(), b, hq, lq, hkv, lk, d, cta_k, q.stride(0), q.stride(1), q.stride(2),
            k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2),
            input_dtype_code, int(use_midpoint_affine), sm_scale, output_dtype_code, o.stride(0),
            o.stride(2), o.stride(1), int(is_causal), stream_ptr))

    def quantize_v_workspace_size(self, batch, kv_heads, k_len, head_dim) -> int:
        return int(self.lib.risa_b200_quantize_v_workspace_size(batch, kv_heads, k_len, head_dim))

    # -- risa_sdpa_prequantized (csrc/bindings.cpp:277-461) -------------------------------------
    @_on_device_of_first_tensor
    def risa_sdpa_prequantized(self, q_int8, k_int8, v_int8, o, q_scale, k_scale, v_scale,
                               v_center, cta_k, sm_scale, output_dtype_code, stream_ptr,
                               attn_mask=None, sparse_row_offsets=None, sparse_block_indices=None,
                               block_mass=None, is_causal=False, lse=None, key_mask_tiles=None):
        (q_int8, k_int8, v_int8, o, q_scale, k_scale, v_scale, v_center, attn_mask,
         sparse_row_offsets, sparse_block_indices, block_mass, lse, key_mask_tiles) = map(
            _t, (q_int8, k_int8, v_int8, o, q_scale, k_scale, v_scale, v_center, attn_mask,
                 sparse_row_offsets, sparse_block_indices, block_mass, lse, key_mask_tiles))
        b, hq, lq, d = q_int8.shape
        hkv, lk = k_int8.shape[1], k_int8.shape[2]
        padded = (lk + cta_k - 1) // cta_k * cta_k
        if v_int8.ndim != 2 or tuple(v_int8.shape) != (b * hkv * d, padded) or \
                tuple(o.shape) != (b, hq, lq, d) or k_int8.shape[0] != b or k_int8.shape[3] != d:
            raise RuntimeError("risa_sdpa_prequantized: incompatible quantized tensor shapes")
        hnd = (lq <= 1 or o.stride(2) == d) and (hq <= 1 or o.stride(1) == lq * d)
        nhd = (hq <= 1 or o.stride(1) == d) and (lq <= 1 or o.stride(2) == hq * d)
        if not (q_int8.is_contiguous() and k_int8.is_contiguous() and v_int8.is_contiguous()) or \
                o.stride(3) != 1 or not (hnd or nhd):
            raise RuntimeError("risa_sdpa_prequantized: quantized tensors must be contiguous and "
                               "output must use HND- or NHD-contiguous storage")
        if lse is not None and (tuple(lse.shape) != (b, hq, lq) or lse.dtype != torch.float32
                                or not lse.is_contiguous()):
            raise RuntimeError(
                "risa_sdpa_prequantized: LSE must be contiguous float32 [batch_size,Hq,query_length]")
        ms = (0, 0, 0, 0)
        mask_code = -1
        if attn_mask is not None:
            if tuple(attn_mask.shape) != (b, hq, lq, lk):
                raise RuntimeError("risa_sdpa_prequantized: attention mask must be expanded to "
                                   "[batch_size,query_heads,query_length,key_length]")
            if attn_mask.dtype not in DTYPE_CODES:
                raise RuntimeError("risa_sdpa_prequantized: attention mask must be bool, float16, "
                                   "bfloat16, or float32")
            mask_code = DTYPE_CODES[attn_mask.dtype]
            ms = attn_mask.stride()
        o_b = hq * lq * d if b <= 1 else o.stride(0)
        o_n = d if lq <= 1 else o.stride(2)
        o_h = lq * d if hq <= 1 else o.stride(1)
        # room for the parts of a split last wave, only for the calls and shapes that take it
        scratch, scratch_bytes = None, 0
        if attn_mask is None and not is_causal and sparse_row_offsets is None and block_mass is None:
            scratch_bytes = int(self.lib.risa_b200_attention_scratch_size(b, hq, lq, lk, d, cta_k))
            if scratch_bytes:
                with torch.cuda.device(q_int8.device), torch.cuda.stream(
                        torch.cuda.ExternalStream(stream_ptr, device=q_int8.device) if stream_ptr
                        else torch.cuda.default_stream(q_int8.device)):
                    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=q_int8.device)
        self._check(self.lib.risa_b200_attention_scratch(
            _ptr(q_int8), _ptr(k_int8), _ptr(v_int8), _ptr(o), _ptr(q_scale), _ptr(k_scale),
            _ptr(v_scale), _ptr(v_center), _ptr(attn_mask), ms[0], ms[1], ms[2], ms[3], mask_code,
            cta_k, b, lq, lk, hq, hkv, d, o_b, o_n, o_h, sm_scale, output_dtype_code,
            _ptr(sparse_row_offsets), _ptr(sparse_block_indices), _ptr(block_mass),
            int(is_causal), _ptr(lse), _ptr(key_mask_tiles), _ptr(scratch), scratch_bytes,
            stream_ptr))

    # -- pattern construction inside the dense pass (no counterpart in the reference module) ------
    def select_scratch_size(self, k_len, cta_k) -> int:
        return int(self.lib.risa_b200_select_scratch_size(k_len, cta_k))

    def select_max_key_tiles(self, cta_k) -> int:
        return int(self.lib.risa_b200_select_max_key_tiles(cta_k))

    @_on_device_of_first_tensor
    def risa_sdpa_select(self, q_int8, k_int8, v_int8, o, q_scale, k_scale, v_scale, v_center,
                         cta_k, sm_scale, output_dtype_code, stream_ptr, theta, scratch, counts,
                         bitmaps, row_totals, attn_mask=None, is_causal=False, block_masses=None):
        b, hq, lq, d = q_int8.shape
        hkv, lk = k_int8.shape[1], k_int8.shape[2]
        ms, mask_code = (0, 0, 0, 0), -1
        if attn_mask is not None:
            ms, mask_code = attn_mask.stride(), DTYPE_CODES[attn_mask.dtype]
        o_b = hq * lq * d if b <= 1 else o.stride(0)
        o_n = d if lq <= 1 else o.stride(2)
        o_h = lq * d if hq <= 1 else o.stride(1)
        self._check(self.lib.risa_b200_attention_select(
            _ptr(q_int8), _ptr(k_int8), _ptr(v_int8), _ptr(o), _ptr(q_scale), _ptr(k_scale),
            _ptr(v_scale), _ptr(v_center), _ptr(attn_mask), ms[0], ms[1], ms[2], ms[3], mask_code,
            cta_k, b, lq, lk, hq, hkv, d, o_b, o_n, o_h, sm_scale, output_dtype_code,
            int(is_causal), float(theta), _ptr(scratch), scratch.numel() * scratch.element_size(),
            _ptr(block_masses), _ptr(counts), _ptr(bitmaps), _ptr(row_totals), stream_ptr))

    @_on_device_of_first_tensor
    def pack_selected(self, counts, bitmaps, row_totals, row_offsets, block_indices, summary,
                      key_blocks, stream_ptr):
        self._check(self.lib.risa_b200_pack_selected(
            _ptr(counts), _ptr(bitmaps), _ptr(row_totals), _ptr(row_offsets), _ptr(block_indices),
            _ptr(summary), counts.numel(), key_blocks, stream_ptr))

    # -- select_retained_mass_csr (csrc/bindings.cpp, sparse_selection.cu) ----------------------
    def retained_mass_selector_workspace_size(self, row_count: int) -> int:
        return int(self.lib.risa_b200_selector_workspace_size(row_count))

    @_on_device_of_first_tensor
    def select_retained_mass_csr(self, sorted_mass, descending_indices, counts, support,
                                 row_totals, row_offsets, block_indices, summary, scan_workspace,
                                 theta, stream_ptr):
        (sorted_mass, descending_indices, counts, support, row_totals, row_offsets, block_indices,
         summary, scan_workspace) = map(
            _t, (sorted_mass, descending_indices, counts, support, row_totals, row_offsets,
                 block_indices, summary, scan_workspace))
        rows, blocks = sorted_mass.shape
        self._check(self.lib.risa_b200_select_retained_mass(
            _ptr(sorted_mass), _ptr(descending_indices), _ptr(counts), _ptr(support),
            _ptr(row_totals), _ptr(row_offsets), _ptr(block_indices), _ptr(summary),
            _ptr(scan_workspace), scan_workspace.numel(), rows, blocks, float(theta), stream_ptr))

    @_on_device_of_first_tensor
    def prepare_key_mask_tiles(self, mask, tiles, tile_size, stream_ptr):
        mask, tiles = _t(mask), _t(tiles)
        if mask.ndim != 4 or mask.stride(2) != 0 or tile_size not in (64, 128):
            raise RuntimeError("prepare_key_mask_tiles requires an expanded broadcast key mask")
        b, h, _, lk = mask.shape
        self._check(self.lib.risa_b200_prepare_key_mask_tiles(
            _ptr(mask), _ptr(tiles), b, h, lk, tile_size, mask.stride(0), mask.stride(1),
            mask.stride(3), DTYPE_CODES[mask.dtype], stream_ptr))

    @_on_device_of_first_tensor
    def risa_lse_shift(self, q, k, anchors, out, scale, stream_ptr):
        q, k, anchors, out = map(_t, (q, k, anchors, out))
        b, hq, lq, d = q.shape
        self._check(self.lib.risa_b200_correct_lse(
            _ptr(q), _ptr(k), _ptr(anchors), _ptr(out), b, hq, k.shape[1], lq, d, q.stride(0),
            q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), scale,
            DTYPE_CODES[q.dtype], stream_ptr))

    def device_status(self) -> None:
        """Raises if the tensor-core kernel recorded an expired wait (synchronises the device)."""
        self._check(self.lib.risa_b200_device_status())

    def set_attention_path(self, path: int) -> int:
        """Kernel family for calls made by the calling thread (0 automatic, 1 row-per-thread, 2 the
        tensor-core kernel with every softmax path compiled in)."""
        return int(self.lib.risa_b200_set_attention_path(path))

    def bounded_wait_self_test(self, limit_ns: int, stream_ptr) -> None:
        self._check(self.lib.risa_b200_bounded_wait_self_test(limit_ns, stream_ptr))


try:
    if getattr(torch.version, "hip", None) or not getattr(torch.version, "cuda", None):
        raise ImportError("RISA Attention requires an NVIDIA CUDA build of PyTorch")
    _ABI = _Native(_LIB_PATH)
    from . import _C  # noqa: E402  (the PyTorch C++ extension; links librisa_b200.so)
except (ImportError, OSError, AttributeError) as error:
    _C = None
    _ABI = None
    _EXTENSION_ERROR = error


_AVAILABLE: dict = {}



_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream_ptr(device: torch.device) -> int:
    """``cudaStream_t`` of the current stream of ``device`` as an integer.  The raw query skips
    the ``torch.cuda.Stream`` object that ``torch.cuda.current_stream`` builds on every call, which
    is a measurable part of a short call's host time."""
    if _RAW_STREAM is not None:
        index = device.index if device.index is not None else torch.cuda.current_device()
        return _RAW_STREAM(index)
    return torch.cuda.current_stream(device).cuda_stream


def is_available(device: torch.device | int | str | None = None) -> bool:
    """True when the library is loaded and ``device`` is a Blackwell datacenter GPU (compute
    capability 10.x; the library holds sm_100a code, which no other family can load)."""
    if _C is None:
        return False
    if isinstance(device, torch.device) and device.type == "cuda" and device.index is not None:
        known = _AVAILABLE.get(device.index)
        if known is None:
            known = _AVAILABLE[device.index] = _probe(device)
        return known
    return _probe(device)


def _probe(device) -> bool:
    if not torch.cuda.is_available():
        return False
    try:
        resolved = None
        if device is not None:
            resolved = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
            if resolved.type != "cuda":
                return False
        return torch.cuda.get_device_capability(resolved)[0] == REQUIRED_COMPUTE_CAPABILITY_MAJOR
    except (AssertionError, RuntimeError, ValueError):
        return False


def require_extension() -> None:
    if _C is None:
        detail = f": {_EXTENSION_ERROR}" if _EXTENSION_ERROR is not None else ""
        raise RuntimeError(f"RISA Attention CUDA library is not available{detail}")
