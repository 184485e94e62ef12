"""ctypes driver for oracle/_ref/librisa_ref.so: the reference project's own CUDA kernels
(compiled unmodified by oracle/build_ref.sh) called through the exception-catching wrappers of
oracle/ref_shim.cpp.  TEST INFRASTRUCTURE ONLY: the bit-exact golden for codes, scales, capture
statistics and tile sets on the GPU, and the "reference kernels on this GPU" timing leg of
bench.py.  Buffer shapes follow the reference's Python runtime
(src/risa_attention/_quantization.py:92-123, _execution.py:64-98, sparse.py:23-48)."""
from __future__ import annotations

import ctypes
import math
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "librisa_ref.so"
_lib = None
c_i32, c_i64, c_f32, c_f64, c_vp, c_sz = (
    ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t)
DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.bool: 3}


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(LIB_PATH))
        sig = {
            "ref_quantize_qk": [c_vp] * 6 + [c_i32] * 10 + [c_i64] * 6 + [c_i32, c_vp, c_vp],
            "ref_quantize_v": [c_vp] * 4 + [c_i32] * 5 + [c_i64] * 3 + [c_i32, c_i32, c_vp],
            "ref_attention": [c_vp] * 9 + [c_i64] * 4 + [c_i32] * 8 + [c_i64] * 12
            + [c_f32, c_i32, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp],
            "ref_select_retained_mass": [c_vp] * 9 + [c_sz, c_i32, c_i32, c_f64, c_vp],
            "ref_prepare_key_mask_tiles": [c_vp, c_vp] + [c_i32] * 4 + [c_i64] * 3 + [c_i32, c_vp],
            "ref_correct_lse": [c_vp] * 4 + [c_i32] * 5 + [c_i64] * 6 + [c_f32, c_i32, c_vp],
        }
        for name, args in sig.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = c_i32, args
        _lib.ref_last_error.restype = ctypes.c_char_p
        _lib.ref_selector_workspace_size.restype = c_sz
        _lib.ref_selector_workspace_size.argtypes = [c_i32]
    return _lib


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _ok(status):
    if status:
        raise RuntimeError("reference: " + lib().ref_last_error().decode())


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def kernel_head_dim(d):
    return 64 if d <= 64 else 128 if d <= 128 else 256


def prequantize(q, k, v, *, cta_k, midpoint_affine=False):
    """q,k,v already padded to the kernel head dim.  Returns a dict of packed tensors."""
    b, hq, lq, d = q.shape
    hkv, lk = k.shape[1], k.shape[2]
    dev = q.device
    padded = -(-lk // cta_k) * cta_k
    out = {
        "q": torch.empty(q.shape, dtype=torch.int8, device=dev),
        "k": torch.empty(k.shape, dtype=torch.int8, device=dev),
        "q_scale": torch.empty(b, hq, -(-lq // 128) * (64 if d == 256 else 32), device=dev),
        "k_scale": torch.empty(b, hkv, -(-lk // cta_k) * 4, device=dev),
        "v": torch.empty(b * hkv * d, padded, dtype=torch.int8, device=dev),
        "v_scale": torch.empty(b * hkv * d, device=dev),
        "v_center": torch.empty(b * hkv * d, device=dev),
        "anchors": torch.empty(b, hkv, dtype=torch.int32, device=dev),
        "cta_k": cta_k,
    }
    warpq = 16 if d == 256 else 32
    _ok(lib().ref_quantize_qk(
        _p(q), _p(out["q"]), _p(out["q_scale"]), _p(k), _p(out["k"]), _p(out["k_scale"]), b, hq,
        lq, hkv, lk, d, 128, warpq, cta_k, cta_k, q.stride(0), q.stride(1), q.stride(2),
        k.stride(0), k.stride(1), k.stride(2), DT[q.dtype], _p(out["anchors"]), _stream(dev)))
    _ok(lib().ref_quantize_v(
        _p(v), _p(out["v"]), _p(out["v_scale"]), _p(out["v_center"]), b, hkv, lk, d, padded,
        v.stride(0), v.stride(1), v.stride(2), DT[v.dtype], int(midpoint_affine), _stream(dev)))
    return out


def attention(pk, *, sm_scale, out_dtype=torch.bfloat16, mask=None, is_causal=False,
              row_offsets=None, block_indices=None, capture=False, want_lse=False,
              key_mask_tiles=None, out=None):
    q, k, v = pk["q"], pk["k"], pk["v"]
    b, hq, lq, d = q.shape
    hkv, lk = k.shape[1], k.shape[2]
    cta_k = pk["cta_k"]
    dev = q.device
    padded = v.shape[1]
    o = torch.empty(b, hq, lq, d, dtype=out_dtype, device=dev) if out is None else out
    lse = torch.empty(b, hq, lq, device=dev) if want_lse else None
    ws = None
    if capture:
        n_q, n_k = -(-lq // 128), -(-lk // cta_k)
        ws = torch.empty(b * hq * n_q * n_k + b * hq * lq * (2 * n_k + 2), device=dev)
    ms = (0, 0, 0, 0) if mask is None else mask.stride()
    _ok(lib().ref_attention(
        _p(q), _p(k), _p(v), _p(o), _p(pk["q_scale"]), _p(pk["k_scale"]), _p(pk["v_scale"]),
        _p(pk["v_center"]), _p(mask), ms[0], ms[1], ms[2], ms[3],
        -1 if mask is None else DT[mask.dtype], cta_k, b, lq, lk, hq, hkv, d,
        hq * lq * d, d, lq * d, hkv * lk * d, d, lk * d, hkv * d * padded, d * padded, padded,
        o.stride(0), o.stride(2), o.stride(1), sm_scale, DT[out_dtype], _p(row_offsets),
        _p(block_indices), _p(ws), int(is_causal), _p(lse), _stream(dev), _p(key_mask_tiles)))
    return {"out": o, "lse": lse, "workspace": ws}


def select_retained_mass(masses, theta):
    rows, tiles = masses.shape
    dev = masses.device
    srt, order = masses.sort(dim=-1, descending=True)
    counts = torch.empty(rows, dtype=torch.int32, device=dev)
    support = torch.empty(rows, tiles, dtype=torch.uint8, device=dev)
    totals = torch.empty(rows, 2, dtype=torch.float64, device=dev)
    offsets = torch.empty(rows + 1, dtype=torch.int32, device=dev)
    storage = torch.empty(rows * tiles, dtype=torch.int32, device=dev)
    summary = torch.empty(3, dtype=torch.float64, device=dev)
    nbytes = lib().ref_selector_workspace_size(rows)
    scratch = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=dev)
    _ok(lib().ref_select_retained_mass(_p(srt), _p(order), _p(counts), _p(support), _p(totals),
                                       _p(offsets), _p(storage), _p(summary), _p(scratch), nbytes,
                                       rows, tiles, float(theta), _stream(dev)))
    sel, tot, nblk = summary.tolist()
    return offsets, storage[: int(nblk)], sel / max(tot, 1e-20)


def key_mask_tiles(mask, tile):
    b, h, _, lk = mask.shape
    tiles = torch.empty(b, h, -(-lk // tile) + 1, dtype=torch.int32, device=mask.device)
    _ok(lib().ref_prepare_key_mask_tiles(_p(mask), _p(tiles), b, h, lk, tile, mask.stride(0),
                                         mask.stride(1), mask.stride(3), DT[mask.dtype],
                                         _stream(mask.device)))
    return tiles


def lse_shift(q, k, anchors, scale):
    b, hq, lq, d = q.shape
    out = torch.empty(b, hq, lq, device=q.device)
    _ok(lib().ref_correct_lse(_p(q), _p(k), _p(anchors), _p(out), b, hq, k.shape[1], lq, d,
                              q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1),
                              k.stride(2), scale, DT[q.dtype], _stream(q.device)))
    return out
