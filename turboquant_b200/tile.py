"""Nibble packing of the paged cache / tile format (turboquant/tile.py:21-54 in the reference):
two 4-bit values per byte, even index in the HIGH nibble."""
from __future__ import annotations

import torch

TILE_TOKENS = 16
TILE_DIMS = 64


@torch.no_grad()
def pack_4bit(indices: torch.Tensor) -> torch.Tensor:
    even = indices[..., 0::2]
    odd = indices[..., 1::2]
    return ((even << 4) | (odd & 0x0F)).to(torch.uint8)


@torch.no_grad()
def unpack_4bit(packed: torch.Tensor, count: int) -> torch.Tensor:
    p = packed.to(torch.int32)
    out = torch.empty(*packed.shape[:-1], packed.shape[-1] * 2, dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = ((p >> 4) & 0x0F).to(torch.uint8)
    out[..., 1::2] = (p & 0x0F).to(torch.uint8)
    return out[..., :count]
