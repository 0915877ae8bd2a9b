"""The reference's CPU path restated in plain torch calls, for timing and cross-checks.

TEST INFRASTRUCTURE ONLY: used by tests/ and by the benchmark's CPU-baseline legs, never by the
shipped package.  The reference's own modules cannot travel to the GPU box, so these functions
restate, call for call, what they do there:

* ``quantize``: ``TurboQuantMSE.quantize`` (turboquant/quantizer.py:77-91) = ``Tensor.norm`` +
  ``clamp`` + division + signs + the butterfly transform of turboquant/hadamard.py:21-42 +
  ``torch.bucketize`` (turboquant/codebook.py:92-98), packed in the cache's nibble order
  (turboquant/tile.py:37-41);
* ``write_kv_cache``: the quantizer on K and V plus the scatter into the paged cache that the
  reference's write op performs (csrc/src/quantize_write_binding.cu:207-269);
* ``decode_attention``: unpack -> centroids -> inverse rotation -> times the fp16 norm -> fp32
  ``softmax(q K^T scale) V`` per sequence, the dequant-attention statement of
  tests/test_fused_integration.py:127-159.

The C oracle (tq_oracle.c) fixes the arithmetic order so that it can be compared bit for bit;
this module is what that order was derived from, and what a user of the reference on a CPU
actually runs.
"""
from __future__ import annotations

import math

import torch


def fwht(y: torch.Tensor) -> torch.Tensor:
    """Normalized Walsh-Hadamard transform along the last axis (a power of two)."""
    d = y.shape[-1]
    lead = y.shape[:-1]
    y = y.reshape(-1, d)
    h = 1
    while h < d:
        y = y.view(-1, d // (2 * h), 2, h)
        y = torch.stack((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), dim=2).reshape(-1, d)
        h *= 2
    return (y * (1.0 / math.sqrt(d))).reshape(*lead, d)


def quantize(x: torch.Tensor, signs: torch.Tensor, boundaries: torch.Tensor):
    """x fp32 [..., d] -> (codes uint8 [..., d/2] with the even dim in the high nibble, norms fp32 [...])."""
    norms = x.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    y = fwht((x / norms) * signs)
    idx = torch.bucketize(y, boundaries)
    packed = ((idx[..., 0::2] << 4) | idx[..., 1::2]).to(torch.uint8)
    return packed, norms.squeeze(-1)


def write_kv_cache(kv_cache: torch.Tensor, key: torch.Tensor, value: torch.Tensor, signs: torch.Tensor,
                   boundaries: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """kv_cache uint8 [2, nb, bs, H, 80]; key / value fp32 [T, H, 128]; slots int64 [T] (negative: skip)."""
    bs = kv_cache.shape[2]
    keep = slot_mapping >= 0
    slots = slot_mapping[keep]
    block, entry = slots // bs, slots % bs
    for i, src in enumerate((key, value)):
        codes, norms = quantize(src[keep], signs, boundaries)
        nh = norms.to(torch.float16).view(torch.uint8).reshape(*norms.shape, 2)
        kv_cache[i, block, entry, :, :64] = codes
        kv_cache[i, block, entry, :, 64:66] = nh
        kv_cache[i, block, entry, :, 66:68] = nh


def dequant_rows(slots: torch.Tensor, signs: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """slots uint8 [..., 80] -> fp32 [..., 128] un-rotated vectors."""
    codes = slots[..., :64]
    idx = torch.stack((codes >> 4, codes & 0x0F), dim=-1).reshape(*codes.shape[:-1], 128).long()
    y = centroids[idx]
    x = fwht(y) * signs
    norms = slots[..., 64:66].contiguous().view(torch.float16).float()
    return x * norms


def decode_attention(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, seq_lens,
                     signs: torch.Tensor, centroids: torch.Tensor, scale: float) -> torch.Tensor:
    """q fp32 [B, Hq, 128] -> out fp32 [B, Hq, 128]: one decode step over the paged quantized cache."""
    B, Hq, D = q.shape
    H = kv_cache.shape[3]
    page = kv_cache.shape[2]
    g = Hq // H
    out = torch.zeros(B, Hq, D)
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            continue
        t = torch.arange(n)
        pages = block_table[b, t // page].long()
        kd = dequant_rows(kv_cache[0, pages, t % page], signs, centroids)      # [n, H, D]
        vd = dequant_rows(kv_cache[1, pages, t % page], signs, centroids)
        qq = q[b].view(H, g, D)
        s = torch.einsum("hgd,nhd->hgn", qq, kd) * scale
        out[b] = torch.einsum("hgn,nhd->hgd", torch.softmax(s, dim=-1), vd).reshape(Hq, D)
    return out
