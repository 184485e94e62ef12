"""Head sharding of one attention call over several GPUs (one process per GPU).

Every unit of the path -- K anchor and K/V quantisation per (batch, kv head), Q groups, attention
CTAs and CSR rows per (batch, query head, query block) -- is independent across heads, so a call is
split over ranks by query head with each rank's KV heads co-located.  When there are more ranks
than KV heads, the query heads of one KV head are split over several ranks and that KV head is
quantised on each of them (the quantisers are deterministic, so the codes are identical).  Nothing
is exchanged on the hot path; ``gather_heads`` reassembles outputs with one all-gather when the
caller wants them on every rank.  The reference is single-GPU and has no counterpart.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """Slice of the head axes owned by one rank."""

    rank: int
    world_size: int
    q_start: int
    q_stop: int
    kv_start: int
    kv_stop: int

    @property
    def q_heads(self) -> int:
        return self.q_stop - self.q_start


def plan_head_shard(q_heads: int, kv_heads: int, rank: int, world_size: int) -> HeadShard:
    """Contiguous query-head range of ``rank`` and the KV heads those query heads read."""
    if q_heads % kv_heads:
        raise ValueError(f"q head count ({q_heads}) must be divisible by k/v head count ({kv_heads})")
    if q_heads % world_size:
        raise ValueError(f"q head count ({q_heads}) must be divisible by the number of ranks ({world_size})")
    per_rank = q_heads // world_size
    group = q_heads // kv_heads
    if per_rank % group and group % per_rank:
        raise ValueError("query heads per rank must be a multiple or a divisor of the GQA group size")
    q_start = rank * per_rank
    q_stop = q_start + per_rank
    return HeadShard(rank, world_size, q_start, q_stop, q_start // group, (q_stop - 1) // group + 1)


def shard_inputs(q, k, v, shard: HeadShard, attn_mask=None):
    """Views of this rank's heads ([B, H, L, D] layout); a mask with a head axis is sliced too."""
    mask = attn_mask
    if attn_mask is not None and attn_mask.ndim == 4 and attn_mask.shape[1] not in (1,):
        mask = attn_mask[:, shard.q_start:shard.q_stop]
    return (q[:, shard.q_start:shard.q_stop], k[:, shard.kv_start:shard.kv_stop],
            v[:, shard.kv_start:shard.kv_stop], mask)


def gather_heads(local: torch.Tensor, group=None, head_dim: int = 1) -> torch.Tensor:
    """All-gather of per-rank outputs (or LSE) along the head axis; every rank gets the full tensor."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=head_dim)


def merge_patterns(local_offsets: torch.Tensor, local_indices: torch.Tensor, batch: int,
                   group=None):
    """Concatenates per-rank CSR supports (rows ordered [batch, local head, query block]) into the
    global row order [batch, head, query block].  Returns (row_offsets, block_indices) on every
    rank; offsets are rebased so they index the concatenated tile list."""
    world = dist.get_world_size(group)
    counts = (local_offsets[1:] - local_offsets[:-1]).to(torch.int32)
    if world == 1:
        return local_offsets, local_indices
    all_counts = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    sizes = torch.tensor([local_indices.numel()], dtype=torch.int64, device=local_indices.device)
    all_sizes = [torch.empty_like(sizes) for _ in range(world)]
    dist.all_gather(all_sizes, sizes, group=group)
    longest = int(max(int(s) for s in all_sizes))
    padded = torch.zeros(longest, dtype=torch.int32, device=local_indices.device)
    padded[: local_indices.numel()] = local_indices
    all_idx = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(all_idx, padded, group=group)
    rows_per_batch = counts.numel() // batch
    count_rows, index_rows = [], []
    for b in range(batch):
        for r in range(world):
            c = all_counts[r][b * rows_per_batch:(b + 1) * rows_per_batch]
            start = int(all_counts[r][: b * rows_per_batch].sum())
            count_rows.append(c)
            index_rows.append(all_idx[r][start:start + int(c.sum())])
    merged_counts = torch.cat(count_rows)
    offsets = torch.zeros(merged_counts.numel() + 1, dtype=torch.int32, device=counts.device)
    offsets[1:] = merged_counts.cumsum(0)
    return offsets, torch.cat(index_rows)
