"""Seeded synthetic workloads of the benchmark specification, shared by ``bench.py`` and the
full-size parity tests.  All tensors are created on ``device`` from one ``torch.Generator`` in a
fixed order (q, k, v, then any extras), so a (generator name, shape, seed) triple names the data.
"""
from __future__ import annotations

import torch


def dense_inputs(seq_len, device, seed=0, q_heads=16, kv_heads=4, head_dim=128, batch=1,
                 dtype=torch.bfloat16, kv_len=None):
    """Dense sweep: i.i.d. N(0,1) drawn in FP32 and rounded to ``dtype``, HND contiguous; q, k, v
    come from the same generator in that order (the reference's benchmarks/common.py:105-131)."""
    g = torch.Generator(device=device).manual_seed(seed)
    kv_len = seq_len if kv_len is None else kv_len
    q = torch.randn(batch, q_heads, seq_len, head_dim, device=device, generator=g).to(dtype)
    k = torch.randn(batch, kv_heads, kv_len, head_dim, device=device, generator=g).to(dtype)
    v = torch.randn(batch, kv_heads, kv_len, head_dim, device=device, generator=g).to(dtype)
    return q, k, v


def block_centroid_inputs(seq_len, device, seed=0, q_heads=16, kv_heads=4, head_dim=128, batch=1):
    """Sparse-reuse workload of the benchmark spec: every 128-token block of a head gets one
    centroid ~ N(0,1) and its tokens are centroid + 0.5 N(0,1) (Q and K); V ~ N(0,1).  Returns
    (q, k, v, generator); the generator continues into :func:`drift`."""
    g = torch.Generator(device=device).manual_seed(seed)

    def blocks(heads):
        centroid = torch.randn(batch, heads, seq_len // 128, 1, head_dim, device=device, generator=g)
        noise = torch.randn(batch, heads, seq_len // 128, 128, head_dim, device=device, generator=g)
        return (centroid + 0.5 * noise).reshape(batch, heads, seq_len, head_dim).bfloat16()

    q, k = blocks(q_heads), blocks(kv_heads)
    v = torch.randn(batch, kv_heads, seq_len, head_dim, device=device, generator=g).bfloat16()
    return q, k, v, g


def video_block_inputs(seq_len, device, seed=0, q_heads=16, kv_heads=4, head_dim=128, batch=1,
                       clusters=2, prototype_norm=8.0):
    """The reference's own sparse-benchmark workload (benchmarks/sparse.py:33-52): N(0,1) q/k/v
    plus, per KV head, ``clusters`` prototypes of norm 8 added to Q and K by 128-token block (block
    index modulo ``clusters``)."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(batch, q_heads, seq_len, head_dim, device=device, generator=g).bfloat16()
    k = torch.randn(batch, kv_heads, seq_len, head_dim, device=device, generator=g).bfloat16()
    v = torch.randn(batch, kv_heads, seq_len, head_dim, device=device, generator=g).bfloat16()
    proto = torch.randn(batch, kv_heads, clusters, head_dim, device=device, generator=g)
    proto *= prototype_norm / proto.norm(dim=-1, keepdim=True)
    cluster = torch.arange(seq_len, device=device).div(128, rounding_mode="floor") % clusters
    q = q + proto.repeat_interleave(q_heads // kv_heads, dim=1)[:, :, cluster].to(q.dtype)
    k = k + proto[:, :, cluster].to(k.dtype)
    return q, k, v, g


def drift(x, generator, kind):
    """Inputs of a later diffusion step: ``"blend"`` = 0.95 x + 0.05 N(0,1) (benchmark spec),
    ``"additive"`` = x + 0.05 N(0,1) (the reference's sparse benchmark)."""
    noise = torch.randn(x.shape, device=x.device, generator=generator)
    if kind == "additive":
        return (x.float() + 0.05 * noise).to(x.dtype)
    return (0.95 * x.float() + 0.05 * noise).to(x.dtype)


def video_dit_inputs(heads, device, seed=0, seq_len=32760, head_dim=128):
    """Video-DiT-shaped self-attention (Hq = Hkv = ``heads``): N(0,1) with a per-channel standard
    deviation ~ U(0.5, 2) and 1 % of the channels (at least one) scaled by 20; 32760 tokens = 21
    latent frames x 30 x 52 patches = 255 full 128-token blocks and one of 120."""
    g = torch.Generator(device=device).manual_seed(seed)

    def make():
        x = torch.randn(1, heads, seq_len, head_dim, device=device, generator=g)
        std = torch.empty(head_dim, device=device).uniform_(0.5, 2.0, generator=g)
        outliers = torch.randperm(head_dim, device=device, generator=g)[: max(1, head_dim // 100)]
        std[outliers] *= 20.0
        return (x * std).bfloat16()

    return make(), make(), make()
