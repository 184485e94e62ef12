"""CPU restatement of the reference's quantised-attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file;
it is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Every function follows the reference project's CUDA code for the path
(file:line given per function) but is written as vectorised PyTorch on CPU
tensors.  FP32 adds / multiplies are ordinary IEEE round-to-nearest ops, fused
multiply-adds are emulated through FP64 (the FP32 x FP32 product is exact in
FP64).  The reference is compiled with ``--use_fast_math`` (csrc/CMakeLists.txt:40):
its ``x / 127.f``, ``1.f / x``, ``ex2``, ``lg2`` lower to the GPU's approximate
units, which no CPU can reproduce bit-for-bit.  This file uses correctly
rounded FP32 results for those, so against a GPU build of the reference:

* Q/K/V INT8 codes may differ by +-1 on a ~1e-4 fraction of elements,
* U8 probability codes may differ by +-1 on a similar fraction,
* scales agree to a few ulp, outputs / LSE to ~1e-3 of the output RMS.

Parity pinning: the pure-integer / power-of-two known-answer cases of the
reference's own tests (tests/cuda/test_value_quantization.py:18-52,
tests/cuda/test_risa_attention.py:20-92, tests/cuda/test_probability_mass.py:21-70,
tests/cuda/test_key_mask_tiles.py:79-103) are reproduced exactly by this file
(see tests/test_oracle_golden.py); random-data codes are pinned on the GPU by
the reference's own kernels compiled into oracle/_ref (bit-exact golden).
"""
from __future__ import annotations

import math

import torch

LOG2E = 1.44269504088896340736
U8_OFFSET = 7.9943534  # csrc/kernels/attention_types.cuh:40
SIGN_WORDS = (0x1035997B, 0x8087F5EE, 0xEE2E4E1A, 0x71132418)  # quantize_qk_impl.cuh:88-100
V_TOKEN_ORDER = (0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15)  # quantize_v_impl.cuh:47-52

f32 = torch.float32
f64 = torch.float64


def _fma(a, b, c):
    """fma.rn.f32 through FP64 (exact product, one extra rounding at ~2^-29 odds)."""
    return (a.to(f64) * b.to(f64) + torch.as_tensor(c).to(f64)).to(f32)


def _f(x):
    return torch.tensor(x, dtype=f32)


def kernel_head_dim(d: int) -> int:
    """src/risa_attention/_execution.py:40-46."""
    return 64 if d <= 64 else 128 if d <= 128 else 256


def select_key_block_size(kernel_d: int, key_length: int, has_row_mask: bool) -> int:
    """src/risa_attention/_validation.py:64-72."""
    return 128 if (not has_row_mask and kernel_d >= 128 and key_length > 1024) else 64


# ----------------------------------------------------------------------------------------
# Rotation (csrc/kernels/quantize_qk_impl.cuh:69-147)
# ----------------------------------------------------------------------------------------
def rotation_mode(kernel_d: int, key_length: int) -> int:
    """quantize_qk_impl.cuh:769-794: 4 = H4 only, 64 = H64, 128 = signed H128, 129 = plain H128."""
    if key_length <= 256:
        return 4
    return {64: 64, 128: 128, 256: 129}[kernel_d]


def _h4(x):
    x0, x1, x2, x3 = x[..., 0::4], x[..., 1::4], x[..., 2::4], x[..., 3::4]
    a0, a1, a2, a3 = x0 + x1, x0 - x1, x2 + x3, x2 - x3
    y = torch.empty_like(x)
    half = _f(0.5)
    y[..., 0::4] = (a0 + a2) * half
    y[..., 1::4] = (a1 + a3) * half
    y[..., 2::4] = (a0 - a2) * half
    y[..., 3::4] = (a1 - a3) * half
    return y


def _butterfly(x, span):
    """One Walsh-Hadamard stage pairing channel c with c^span: (lo+hi, lo-hi)."""
    shape = x.shape
    v = x.reshape(*shape[:-1], shape[-1] // (2 * span), 2, span)
    lo, hi = v[..., 0, :], v[..., 1, :]
    return torch.stack((lo + hi, lo - hi), dim=-2).reshape(shape)


def rotate(x: torch.Tensor, mode: int) -> torch.Tensor:
    """x: [..., D] float32 (D = 64/128/256).  Stage order: channel bits 1,2 (H4, x0.5), then
    4,8,16,32(,64), then the final normalisation multiply (quantize_qk_impl.cuh:106-142)."""
    x = x.to(f32)
    if mode == 4:
        return _h4(x)
    if mode == 64:
        y = _h4(x)
        for span in (4, 8, 16, 32):
            y = _butterfly(y, span)
        return y * _f(0.25)
    d = x.shape[-1]
    tiles = x.reshape(*x.shape[:-1], d // 128, 128)
    if mode == 128:
        bits = torch.tensor(
            [((SIGN_WORDS[i // 32] >> (i % 32)) & 1) for i in range(128)], dtype=torch.bool
        )
        tiles = torch.where(bits, tiles, -tiles)  # negate where the bit is 0
    y = _h4(tiles)
    for span in (4, 8, 16, 32, 64):
        y = _butterfly(y, span)
    y = y * _f(0.1767766952966369)
    return y.reshape(x.shape)


def _to_codes(v, inv):
    """cvt.rni.sat.s8.f32(v * inv) (csrc/float_utils.cuh:23-31)."""
    return torch.clamp(torch.round(v * inv), -128, 127).to(torch.int8)


# ----------------------------------------------------------------------------------------
# K anchor (quantize_qk_impl.cuh:442-577)
# ----------------------------------------------------------------------------------------
def detect_k_anchor(k: torch.Tensor) -> torch.Tensor:
    """k: [B,Hkv,Lk,D] float32 -> int32 [B,Hkv] absolute row index or -1.

    The thread/warp summation tree of the reference (thread t owns channels t, t+128; shfl_down
    tree; warps added 0..3) is reproduced so the strict comparisons see the same FP32 sums."""
    b_, h_, lk, d = k.shape
    out = torch.empty(b_, h_, dtype=torch.int32)
    rows = [s * (lk - 1) // 8 for s in range(9)]
    for b in range(b_):
        for h in range(h_):
            smp = k[b, h, rows].to(f32)  # [9, D]
            ch = torch.full((9, 256), 0.0, dtype=f32)
            ch[:, :d] = smp
            act = torch.zeros(256, dtype=torch.bool)
            act[:d] = True

            energy = torch.zeros(128, dtype=f32)
            omax = torch.zeros(128, dtype=f32)
            dist = torch.zeros(9, 128, dtype=f32)
            for base in range(0, d, 128):
                n = min(128, d - base)
                vals = ch[:, base : base + n]  # [9, n]
                csum = torch.zeros(n, dtype=f32)
                e = energy[:n].clone()
                m = omax[:n].clone()
                for s in range(9):
                    e = _fma(vals[s], vals[s], e)
                    m = torch.maximum(m, vals[s].abs())
                    csum = csum + vals[s]
                energy[:n] = e
                omax[:n] = m
                for c in range(9):
                    dd = _fma(_f(9.0), vals[c], -csum)
                    dist[c, :n] = _fma(dd, dd, dist[c, :n])

            def warp_tree_sum(x128):  # shfl_down tree per warp then warps 0..3 in order
                w = x128.reshape(4, 32).clone()
                for off in (16, 8, 4, 2, 1):
                    sh = torch.zeros_like(w)
                    sh[:, : 32 - off] = w[:, off:]
                    sh[:, 32 - off :] = w[:, 32 - off :]  # out-of-range lanes read themselves
                    w = w + sh
                tot = _f(0.0)
                for i in range(4):
                    tot = tot + w[i, 0]
                return tot

            def warp_tree_max(x128):
                return x128.max()

            total_energy = warp_tree_sum(energy)
            total_max = warp_tree_max(omax)
            best_c, best_d = 0, _f(3.402823466e38)
            for c in range(9):
                dc = warp_tree_sum(dist[c])
                if dc < best_d:
                    best_c, best_d = c, dc
            be = torch.zeros(128, dtype=f32)
            bm = torch.zeros(128, dtype=f32)
            for base in range(0, d, 128):
                n = min(128, d - base)
                vals = ch[:, base : base + n]
                e = be[:n].clone()
                m = bm[:n].clone()
                for s in range(9):
                    r = vals[s] - vals[best_c]
                    e = _fma(r, r, e)
                    m = torch.maximum(m, r.abs())
                be[:n] = e
                bm[:n] = m
            best_energy = warp_tree_sum(be)
            best_max = warp_tree_max(bm)
            ok = bool(best_energy < total_energy) and bool(best_max <= total_max * _f(1.125))
            out[b, h] = rows[best_c] if ok else -1
    return out


# ----------------------------------------------------------------------------------------
# Q / K quantisation (quantize_qk_impl.cuh:153-426)
# ----------------------------------------------------------------------------------------
def _group_scale(mx):
    sc = mx / _f(127.0) + _f(1e-7)  # div.approx + add on the GPU
    return sc, _f(1.0) / sc  # rcp.approx on the GPU


def quantize_q(q: torch.Tensor, key_length: int):
    """q: [B,Hq,Lq,D] (D in 64/128/256).  Returns codes int8 [B,Hq,Lq,D] and scales f32
    [B,Hq,ceil(Lq/128)*(32|64)].  Group of row n: (n/32)*8+n%8 for D<=128, (n/16)*8+n%8 for D=256
    (quantize_qk_impl.cuh:158-166,236)."""
    b_, h_, lq, d = q.shape
    mode = rotation_mode(d, key_length)
    warpq = 16 if d == 256 else 32
    per_block = 128 // warpq * 8
    nblk = (lq + 127) // 128
    lpad = nblk * 128
    x = torch.zeros(b_, h_, lpad, d, dtype=f32)
    x[:, :, :lq] = rotate(q.to(f32), mode)
    # rows of a warp tile: [tile, j, g] with n = tile*warpq + j*8 + g
    t = x.reshape(b_, h_, lpad // warpq, warpq // 8, 8, d)
    mx = t.abs().amax(dim=(3, 5))  # [B,H,tiles,8]
    sc, inv = _group_scale(mx)
    codes = _to_codes(t, inv[:, :, :, None, :, None]).reshape(b_, h_, lpad, d)[:, :, :lq]
    scales = sc.reshape(b_, h_, nblk * per_block)
    return codes.contiguous(), scales.contiguous()


def quantize_k(k: torch.Tensor, cta_k: int, anchors: torch.Tensor | None = None):
    """k: [B,Hkv,Lk,D].  Group of row n: (n/cta_k)*4 + (n%8)/2 (quantize_qk_impl.cuh:325,388).
    The anchor row (raw input) is subtracted before rotation (:292-307,330-332)."""
    b_, h_, lk, d = k.shape
    mode = rotation_mode(d, lk)
    x = k.to(f32)
    if anchors is not None:
        idx = anchors.clamp_min(0).long()
        rows = torch.gather(x, 2, idx[..., None, None].expand(b_, h_, 1, d))
        rows = rows * (anchors >= 0)[..., None, None].to(f32)
        x = x - rows
    nblk = (lk + cta_k - 1) // cta_k
    lpad = nblk * cta_k
    r = torch.zeros(b_, h_, lpad, d, dtype=f32)
    r[:, :, :lk] = rotate(x, mode)
    t = r.reshape(b_, h_, nblk, cta_k // 8, 4, 2, d)
    mx = t.abs().amax(dim=(3, 5, 6))  # [B,H,nblk,4]
    sc, inv = _group_scale(mx)
    codes = _to_codes(t, inv[:, :, :, None, :, None, None]).reshape(b_, h_, lpad, d)[:, :, :lk]
    return codes.contiguous(), sc.reshape(b_, h_, nblk * 4).contiguous()


# ----------------------------------------------------------------------------------------
# V quantisation (csrc/kernels/quantize_v_impl.cuh:83-292)
# ----------------------------------------------------------------------------------------
def quantize_v(v: torch.Tensor, cta_k: int, midpoint_affine: bool):
    """v: [B,Hkv,Lk,D] -> codes int8 [B*Hkv*D, padded_Lk] (token-permuted, zero tail), scale and
    centre f32 [B*Hkv*D].  The midpoint-affine residual is summed in the reference's order:
    thread t of 512 (128 if Lk<=256) visits tokens Lk-1-t, Lk-1-t-512, ...; xor-butterfly inside
    each warp; warps added in index order (quantize_v_impl.cuh:233-275)."""
    b_, h_, lk, d = v.shape
    x = v.to(f32)
    padded = (lk + cta_k - 1) // cta_k * cta_k
    if midpoint_affine:
        mn, mx = x.amin(2), x.amax(2)
        center = _f(0.5) * (mn + mx)
        radius = _f(0.5) * (mx - mn)
    else:
        mx = x.abs().amax(2)
        center = torch.zeros_like(mx)
        radius = mx
    sc = torch.maximum(radius * _f(1.0 / 127.0), _f(1e-12))
    inv = _f(1.0) / sc
    norm = (x - center[:, :, None, :]) * inv[:, :, None, :]
    codes = torch.clamp(torch.round(norm), -128, 127)
    out_center = center
    if midpoint_affine:
        threads = 128 if lk <= 256 else 512
        res = norm - codes  # [B,H,Lk,D]
        steps = (lk + threads - 1) // threads
        rev = torch.zeros(b_, h_, steps * threads, d, dtype=f32)
        rev[:, :, :lk] = res.flip(2)  # position p <-> token Lk-1-p ; thread = p % threads
        rev = rev.reshape(b_, h_, steps, threads, d)
        acc = torch.zeros(b_, h_, threads, d, dtype=f32)
        for i in range(steps):
            acc = acc + rev[:, :, i]
        w = acc.reshape(b_, h_, threads // 32, 32, d)
        for off in (16, 8, 4, 2, 1):
            idx = torch.arange(32) ^ off
            w = w + w[:, :, :, idx]
        total = torch.zeros(b_, h_, d, dtype=f32)
        for i in range(threads // 32):
            total = total + w[:, :, i, 0]
        scale_back = _f(1.0) / inv
        out_center = _fma(scale_back, total / _f(float(lk)), center)
    packed = torch.zeros(b_, h_, d, padded, dtype=torch.int8)
    packed[..., :lk] = codes.to(torch.int8).transpose(2, 3)
    order = torch.tensor(V_TOKEN_ORDER)
    packed = packed.reshape(b_, h_, d, padded // 16, 16)[..., order].reshape(b_ * h_ * d, padded)
    return packed.contiguous(), sc.reshape(-1).contiguous(), out_center.reshape(-1).contiguous()


def unpermute_v(packed: torch.Tensor) -> torch.Tensor:
    """[rows, padded] storage order -> token order."""
    rows, padded = packed.shape
    inv = torch.empty(16, dtype=torch.long)
    inv[torch.tensor(V_TOKEN_ORDER)] = torch.arange(16)
    return packed.reshape(rows, padded // 16, 16)[..., inv].reshape(rows, padded)


# ----------------------------------------------------------------------------------------
# LSE shift (csrc/kernels/lse_correction.cu:4-28)
# ----------------------------------------------------------------------------------------
def lse_shift(q, k, anchors, scale):
    b_, hq, lq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    out = torch.zeros(b_, hq, lq, dtype=f32)
    for b in range(b_):
        for h in range(hq):
            a = int(anchors[b, h // g])
            if a < 0:
                continue
            prod = q[b, h].to(f32) * k[b, h // g, a].to(f32)[None, :]  # [Lq, D]
            lanes = torch.zeros(lq, 32, dtype=f32)
            for base in range(0, d, 32):
                lanes = lanes + prod[:, base : base + 32]
            for off in (16, 8, 4, 2, 1):
                sh = lanes.clone()
                sh[:, : 32 - off] = lanes[:, off:]
                lanes = lanes + sh
            out[b, h] = lanes[:, 0] * _f(scale)
    return out


# ----------------------------------------------------------------------------------------
# Broadcast key-mask tiles (csrc/kernels/key_mask_tiles.cu:10-43)
# ----------------------------------------------------------------------------------------
def key_mask_tiles(mask: torch.Tensor, tile: int) -> torch.Tensor:
    """mask: [B,Hq,1|Lq,Lk] broadcast over queries.  Returns int32 [B,Hq,tiles+1]: visible tile
    ids compacted to the front, the count in the last slot; the remaining slots keep the 0/1
    'excluded' flags the reference leaves there."""
    b_, h_, _, lk = mask.shape
    n = (lk + tile - 1) // tile
    row = mask[:, :, 0]
    vis = row if row.dtype == torch.bool else torch.isfinite(row.float())
    pad = torch.zeros(b_, h_, n * tile, dtype=torch.bool)
    pad[..., :lk] = vis
    tile_vis = pad.reshape(b_, h_, n, tile).any(-1)
    out = torch.zeros(b_, h_, n + 1, dtype=torch.int32)
    out[..., :n] = (~tile_vis).to(torch.int32)
    for b in range(b_):
        for h in range(h_):
            ids = torch.nonzero(tile_vis[b, h]).flatten().to(torch.int32)
            out[b, h, : ids.numel()] = ids
            out[b, h, n] = ids.numel()
    return out


# ----------------------------------------------------------------------------------------
# Fused attention (csrc/kernels/attention_int8.cuh:145-1026, attention_softmax.cuh,
# attention_value.cuh, attention_masks.cuh)
# ----------------------------------------------------------------------------------------
def _exp2(x):
    return torch.exp2(x.to(f64)).to(f32)


def _rni_u8(p):
    return torch.clamp(torch.round(p), 0, 255)


def attention(
    q_codes,
    k_codes,
    v_packed,
    q_scale,
    k_scale,
    v_scale,
    v_center,
    *,
    cta_k: int,
    sm_scale: float,
    mask: torch.Tensor | None = None,
    is_causal: bool = False,
    row_offsets: torch.Tensor | None = None,
    block_indices: torch.Tensor | None = None,
    capture: bool = False,
    want_lse: bool = False,
    out_dtype=torch.bfloat16,
    heads=None,
    q_blocks=None,
):
    """Returns dict(out=[B,Hq,Lq,D] out_dtype, lse=[B,Hq,Lq] f32|None, workspace=f32|None).

    One 128-query block of one (batch, head) at a time; key tiles visited in order, the last
    visited tile through the generic path (attention_int8.cuh:721-865).  ``heads`` / ``q_blocks``
    restrict the computation to a subset (used to bound the timed CPU sample)."""
    b_, hq, lq, d = q_codes.shape
    hkv, lk = k_codes.shape[1], k_codes.shape[2]
    g = hq // hkv
    n_k = (lk + cta_k - 1) // cta_k
    n_q = (lq + 127) // 128
    padded = n_k * cta_k
    warpq = 16 if d == 256 else 32
    q_per_blk = 128 // warpq * 8
    v_tok = unpermute_v(v_packed).reshape(b_, hkv, d, padded).to(f32)
    scale2 = _f(sm_scale) * _f(LOG2E)
    fast = mask is None and not is_causal and sm_scale > 0
    prescale = not fast
    key_mask = mask is not None and mask.stride(-2) == 0
    out = torch.zeros(b_, hq, lq, d, dtype=out_dtype)
    lse = torch.full((b_, hq, lq), float("nan"), dtype=f32) if want_lse else None
    ws = None
    if capture:
        rows_total = b_ * hq * lq
        mass_elems = b_ * hq * n_q * n_k
        ws = torch.zeros(mass_elems + rows_total * (2 * n_k + 2), dtype=f32)
        ws_i = ws.view(torch.int32)
        full_words = rows_total * (n_k - 1) * 2
    col = torch.arange(cta_k)
    grp = (col % 8) // 2  # K scale group of a key column
    lane_q = grp  # quad lane owning the column
    t16 = col // 16
    for b in range(b_):
        for h in range(hq) if heads is None else heads:
            kh = h // g
            for bx in range(n_q) if q_blocks is None else q_blocks:
                r0, r1 = bx * 128, min(lq, bx * 128 + 128)
                nr = r1 - r0
                rows = torch.arange(r0, r1)
                qi = q_codes[b, h, r0:r1].to(f32)
                qg = (rows // warpq) * 8 + rows % 8
                qs = q_scale[b, h, qg]  # [nr]
                if row_offsets is not None:
                    row = (b * hq + h) * n_q + bx
                    tiles = block_indices[int(row_offsets[row]) : int(row_offsets[row + 1])].tolist()
                elif is_causal and not capture:
                    tiles = list(range((min(lk, (bx + 1) * 128) + cta_k - 1) // cta_k))
                else:
                    tiles = list(range(n_k))
                m = torch.full((nr,), -50000.0, dtype=f32)
                dpart = torch.zeros(nr, 4, dtype=f32)
                o = torch.zeros(nr, d, dtype=f32)
                for it, t in enumerate(tiles):
                    last = it == len(tiles) - 1
                    c0 = t * cta_k
                    kt = torch.zeros(cta_k, d, dtype=f32)
                    nk = max(0, min(cta_k, lk - c0))
                    kt[:nk] = k_codes[b, kh, c0 : c0 + nk].to(f32)
                    s = qi @ kt.T  # exact integers in fp32
                    ks = k_scale[b, kh, t * 4 : t * 4 + 4]  # [4]
                    sc = scale2 * (qs[:, None] * ks[None, :])  # [nr,4]
                    sc_col = sc[:, grp]  # [nr,cta_k]
                    kv_idx = c0 + col
                    if prescale:
                        x = s * sc_col
                        if mask is not None:
                            mt = mask[b, h, 0 if key_mask else slice(r0, r1)]
                            mt = mt[..., c0 : c0 + nk]
                            if key_mask:
                                mt = mt[None, :].expand(nr, nk)
                            keep = torch.zeros(nr, cta_k, dtype=torch.bool)
                            bias = torch.zeros(nr, cta_k, dtype=f32)
                            if mt.dtype == torch.bool:
                                keep[:, :nk] = mt
                            else:
                                bias[:, :nk] = mt.to(f32)
                                keep[:, :nk] = torch.isfinite(bias[:, :nk])
                            x = torch.where(keep, x + bias * _f(LOG2E), _f(-math.inf))
                        if is_causal:
                            x = torch.where(kv_idx[None, :] > rows[:, None], _f(-math.inf), x)
                        if last:
                            x = torch.where(kv_idx[None, :] >= lk, _f(-math.inf), x)
                        # per-lane (column group) max starts at -50000
                        gm = torch.stack(
                            [x[:, grp == w].amax(1) for w in range(4)], 1
                        ).clamp_min(-50000.0)
                        tile_m = (gm - _f(U8_OFFSET)).amax(1)
                        p = _exp2(x + (-tile_m)[:, None])
                    else:
                        x = s
                        if last:
                            x = torch.where(kv_idx[None, :] >= lk, _f(-1.0e30), x)
                            gm = torch.stack(
                                [x[:, grp == w].amax(1) for w in range(4)], 1
                            ).clamp_min(-50000.0)
                        else:
                            gm = torch.stack([x[:, grp == w].amax(1) for w in range(4)], 1)
                        tile_m = _fma(gm, sc, -U8_OFFSET).amax(1)
                        p = _exp2(_fma(x, sc_col, (-tile_m)[:, None]))
                    pu = _rni_u8(p)
                    m_prev = m
                    m = torch.maximum(m_prev, tile_m)
                    e = _exp2(-(m_prev - tile_m).abs())
                    o_scale = torch.where(m_prev < tile_m, e, _f(1.0))
                    w = torch.where(tile_m < m_prev, e, _f(1.0))
                    dprev = dpart
                    dpart = dpart * o_scale[:, None]
                    # denominator partials: lane q owns columns with (c%8)/2 == q
                    for lane in range(4):
                        sel = pu[:, lane_q == lane].reshape(nr, cta_k // 16, 4)
                        if last:
                            s8 = sel.reshape(nr, cta_k // 32, 8).sum(-1)
                            # the compiled reference fuses the rescale with the first addend:
                            # d * o_scale + round(s * w) in one FMA (found on the GPU, bit for bit)
                            dpart[:, lane] = _fma(dprev[:, lane], o_scale, s8[:, 0] * w)
                            for j in range(1, cta_k // 32):
                                dpart[:, lane] = _fma(s8[:, j], w, dpart[:, lane])
                        else:
                            s4 = sel.sum(-1)
                            for j in range(cta_k // 16):
                                dpart[:, lane] = _fma(s4[:, j], w, dpart[:, lane])
                    o = o * o_scale[:, None]
                    acc = pu @ v_tok[b, kh, :, c0 : c0 + cta_k].T  # exact integers
                    o = _fma(acc, w[:, None], o)
                    if capture:
                        grow = (b * hq + h) * lq + rows
                        numer = pu.sum(1)
                        if last:
                            base = mass_elems + full_words + grow * 2
                            ws[base] = numer
                            ws[base + 1] = tile_m
                        else:
                            base = mass_elems + (grow * (n_k - 1) + it) * 2
                            ws_i[base] = numer.to(torch.int32)
                            ws[base + 1] = tile_m
                dsum = (dpart[:, 0] + dpart[:, 1]) + (dpart[:, 2] + dpart[:, 3])
                if capture:
                    grow = (b * hq + h) * lq + rows
                    base = mass_elems + full_words + rows_total * 2 + grow * 2
                    ws[base] = m
                    ws[base + 1] = dsum
                res = o * (_f(1.0) / dsum)[:, None]
                vs = v_scale[(b * hkv + kh) * d : (b * hkv + kh + 1) * d]
                vc = v_center[(b * hkv + kh) * d : (b * hkv + kh + 1) * d]
                res = _fma(res, vs[None, :], vc[None, :])
                if mask is not None or is_causal:
                    res = torch.where((dsum > 0)[:, None], res, _f(0.0))
                out[b, h, r0:r1] = res.to(out_dtype)
                if want_lse:
                    val = (torch.log2(dsum.to(f64)).to(f32) + m) / _f(LOG2E)
                    lse[b, h, r0:r1] = torch.where(dsum > 0, val, _f(-math.inf))
    if capture:
        _block_masses(ws, b_, hq, lq, n_q, n_k)
    return {"out": out, "lse": lse, "workspace": ws}


def _block_masses(ws, b_, hq, lq, n_q, n_k):
    """captured_block_mass_kernel (attention_int8.cuh:1028-1088): shfl_down trees."""
    rows_total = b_ * hq * lq
    mass_elems = b_ * hq * n_q * n_k
    ws_i = ws.view(torch.int32)
    full_words = rows_total * (n_k - 1) * 2
    st = mass_elems + full_words + rows_total * 2
    m_fin = ws[st : st + rows_total * 2 : 2]
    d_fin = ws[st + 1 : st + rows_total * 2 : 2]
    for bh in range(b_ * hq):
        for bx in range(n_q):
            r0, r1 = bx * 128, min(lq, bx * 128 + 128)
            grow = bh * lq + torch.arange(r0, r1)
            for t in range(n_k):
                if t + 1 < n_k:
                    base = mass_elems + (grow * (n_k - 1) + t) * 2
                    numer = ws_i[base].to(f32)
                else:
                    base = mass_elems + full_words + grow * 2
                    numer = ws[base]
                tmax = ws[base + 1]
                qm = torch.where(
                    d_fin[grow] > 0,
                    numer * _exp2(tmax - m_fin[grow]) / d_fin[grow],
                    _f(0.0),
                )
                full = torch.zeros(128, dtype=f32)
                full[: r1 - r0] = qm
                wv = full.reshape(4, 32)
                for off in (16, 8, 4, 2, 1):
                    sh = wv.clone()
                    sh[:, : 32 - off] = wv[:, off:]
                    wv = wv + sh
                lanes = torch.zeros(32, dtype=f32)
                lanes[:4] = wv[:, 0]
                for off in (16, 8, 4, 2, 1):
                    sh = lanes.clone()
                    sh[: 32 - off] = lanes[off:]
                    lanes = lanes + sh
                ws[(bh * n_q + bx) * n_k + t] = lanes[0]


# ----------------------------------------------------------------------------------------
# Retained-mass selection (src/risa_attention/sparse.py:18-52, csrc/kernels/sparse_selection.cu)
# ----------------------------------------------------------------------------------------
def select_retained_mass(masses: torch.Tensor, theta: float):
    """masses f32 [R,n] -> (row_offsets int32 [R+1], block_indices int32 [N], measured_mass)."""
    r_, n = masses.shape
    srt, idx = masses.sort(dim=-1, descending=True)
    counts = torch.empty(r_, dtype=torch.int64)
    sel_sum = torch.zeros(r_, dtype=f64)
    tot_sum = torch.zeros(r_, dtype=f64)
    sd = srt.to(f64)
    npad = (n + 31) // 32 * 32
    padded = torch.zeros(r_, npad, dtype=f64)
    padded[:, :n] = sd
    lanes = padded.reshape(r_, npad // 32, 32)
    lane_tot = torch.zeros(r_, 32, dtype=f64)
    for c in range(npad // 32):
        lane_tot = lane_tot + lanes[:, c]
    for off in (16, 8, 4, 2, 1):
        sh = lane_tot.clone()
        sh[:, : 32 - off] = lane_tot[:, off:]
        lane_tot = lane_tot + sh
    total = lane_tot[:, 0]
    target = theta * total
    cumulative = torch.zeros(r_, dtype=f64)
    done = torch.zeros(r_, dtype=torch.bool)
    counts[:] = n
    sel_sum[:] = total
    lane_id = torch.arange(32)
    for c in range(npad // 32):
        pre = lanes[:, c].clone()
        for off in (1, 2, 4, 8, 16):
            prev = torch.zeros_like(pre)
            prev[:, off:] = pre[:, : 32 - off]
            pre = torch.where(lane_id[None, :] >= off, pre + prev, pre)
        rank = c * 32 + lane_id
        reach = (rank[None, :] < n) & (cumulative[:, None] + pre >= target[:, None])
        anyr = reach.any(1) & ~done
        first = reach.to(torch.int8).argmax(1)
        counts = torch.where(anyr, c * 32 + first + 1, counts)
        sel_sum = torch.where(anyr, cumulative + pre.gather(1, first[:, None])[:, 0], sel_sum)
        done |= anyr
        cumulative = cumulative + pre[:, 31]
    tot_sum = total
    offsets = torch.zeros(r_ + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    chosen = []
    for r in range(r_):
        chosen.append(idx[r, : int(counts[r])].sort().values.to(torch.int32))
    block_indices = torch.cat(chosen) if chosen else torch.zeros(0, dtype=torch.int32)
    # finalize_offsets_and_summary_kernel: 256 strided partials then a halving tree
    def tree(x):
        part = torch.zeros(256, dtype=f64)
        for r0 in range(0, r_, 256):
            seg = x[r0 : r0 + 256]
            part[: seg.numel()] = part[: seg.numel()] + seg
        stride = 128
        while stride > 0:
            part[:stride] = part[:stride] + part[stride : 2 * stride]
            stride //= 2
        return float(part[0])

    measured = tree(sel_sum) / max(tree(tot_sum), 1e-20)
    return offsets, block_indices, measured


# ----------------------------------------------------------------------------------------
# End-to-end helpers mirroring the Python runtime (src/risa_attention/_quantization.py,
# _execution.py, sparse.py)
# ----------------------------------------------------------------------------------------
def prequantize(q, k, v, *, scale=None, attn_mask=None, v_quantization="absmax"):
    d0 = q.shape[-1]
    kd = kernel_head_dim(d0)
    if kd != d0:
        pad = (0, kd - d0)
        q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
    b_, hq, lq, _ = q.shape
    lk = k.shape[2]
    if attn_mask is not None:
        attn_mask = torch.broadcast_to(attn_mask, (b_, hq, lq, lk))
    has_row_mask = attn_mask is not None and attn_mask.stride(-2) != 0
    cta_k = select_key_block_size(kd, lk, has_row_mask)
    anchors = detect_k_anchor(k.float())
    qc, qs = quantize_q(q.float(), lk)
    kc, ks = quantize_k(k.float(), cta_k, anchors)
    vc, vs, vcen = quantize_v(v.float(), cta_k, v_quantization == "midpoint_affine")
    return {
        "q": qc, "k": kc, "v": vc, "q_scale": qs, "k_scale": ks, "v_scale": vs, "v_center": vcen,
        "anchors": anchors, "cta_k": cta_k, "scale": d0**-0.5 if scale is None else float(scale),
        "mask": attn_mask, "head_dim": d0, "q_in": q, "k_in": k,
    }


def int8_attention(q, k, v, *, scale=None, attn_mask=None, v_quantization="absmax",
                   is_causal=False, return_lse=False, out_dtype=None):
    pk = prequantize(q, k, v, scale=scale, attn_mask=attn_mask, v_quantization=v_quantization)
    if out_dtype is None:
        out_dtype = torch.bfloat16 if q.dtype == torch.float32 else q.dtype
    r = attention(pk["q"], pk["k"], pk["v"], pk["q_scale"], pk["k_scale"], pk["v_scale"],
                  pk["v_center"], cta_k=pk["cta_k"], sm_scale=pk["scale"], mask=pk["mask"],
                  is_causal=is_causal, want_lse=return_lse, out_dtype=out_dtype)
    out = r["out"][..., : pk["head_dim"]]
    out = out.float() if q.dtype == torch.float32 else out
    if return_lse:
        return out, r["lse"] + lse_shift(pk["q_in"].float(), pk["k_in"].float(), pk["anchors"], pk["scale"])
    return out


def sdpa_fp32(q, k, v, *, scale=None, attn_mask=None, is_causal=False):
    """FP32 accuracy reference (benchmarks/common.py:134-145 semantics, unchunked)."""
    q, k, v = q.float(), k.float(), v.float()
    g = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    sc = q.shape[-1] ** -0.5 if scale is None else scale
    s = (q @ k.transpose(-1, -2)) * sc
    if attn_mask is not None:
        s = s.masked_fill(~attn_mask, -math.inf) if attn_mask.dtype == torch.bool else s + attn_mask.float()
    if is_causal:
        lq, lk = s.shape[-2:]
        s = s.masked_fill(torch.arange(lk)[None, :] > torch.arange(lq)[:, None], -math.inf)
    lse = torch.logsumexp(s, -1)
    return (s.softmax(-1).nan_to_num(nan=0.0) @ v), lse
