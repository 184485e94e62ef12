"""Seeded input generators and comparison helpers shared by the tests."""
from __future__ import annotations

import torch


def qkv(b, hq, hkv, lq, lk, d, dtype, seed=0, device="cuda", anchor=False, layout="hnd"):
    g = torch.Generator(device=device).manual_seed(seed)
    def make(h, n):
        if layout == "nhd":
            return torch.randn(b, n, h, d, generator=g, device=device, dtype=torch.float32).to(dtype).transpose(1, 2)
        return torch.randn(b, h, n, d, generator=g, device=device, dtype=torch.float32).to(dtype)
    q, k, v = make(hq, lq), make(hkv, lk), make(hkv, lk)
    if anchor:  # clustered keys: subtracting a sampled key shrinks the range, the anchor fires
        k = (k.float() * 0.1 + 4).to(dtype)
    return q, k, v


def pad_to_kernel_dim(x):
    d = x.shape[-1]
    kd = 64 if d <= 64 else 128 if d <= 128 else 256
    return x if kd == d else torch.nn.functional.pad(x, (0, kd - d))


def rel_max_err(a, b):
    """max |a-b| relative to the RMS of b."""
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt().clamp_min(1e-12)
    return ((a - b).abs().max() / rms).item()


def nrmse(a, b):
    a, b = a.float(), b.float()
    return ((a - b).pow(2).mean() / b.pow(2).mean().clamp_min(1e-30)).sqrt().item()


def assert_outputs_match(ours, ref, tol=2e-3):
    """Output parity rule: |ours - ref| <= tol * RMS(ref) + one unit in the last place of the
    16-bit output type.  The FP32 results must agree to ``tol`` of the output RMS; the final
    rounding to bf16/fp16 (8 / 11 significant bits) may then land on the neighbouring value."""
    a, b = ours.float(), ref.float()
    rms = b.pow(2).mean().sqrt()
    eps = 2.0 ** -7 if ref.dtype == torch.bfloat16 else 2.0 ** -10
    ulp = torch.maximum(b.abs(), a.abs()) * eps
    bad = (a - b).abs() > tol * rms + ulp
    assert not bad.any(), f"{int(bad.sum())} outputs beyond tolerance, worst {((a - b).abs() / rms).max().item():.3e} x RMS"
