"""Visible-tile lists for masks that are broadcast over queries, so the kernel can skip key tiles
with no visible key (reference src/risa_attention/_key_mask.py:9-28)."""
import torch

from . import _backend


def prepare_key_mask_tiles(mask, key_block_size, query_length, scale, is_causal):
    if mask is None or mask.stride(-2) != 0 or mask.shape[-1] <= 1024 or query_length < 256 \
            or scale <= 0 or is_causal:
        return None
    batch, heads, _, length = mask.shape
    tiles = torch.empty((batch, heads, -(-length // key_block_size) + 1), device=mask.device,
                        dtype=torch.int32)
    _backend._C.prepare_key_mask_tiles(mask, tiles, key_block_size,
                                       _backend.current_stream_ptr(mask.device))
    return tiles
