"""Lloyd-Max codebook with the reference's interface (turboquant/codebook.py:65-103).

Centroids and boundaries come from the library's host-side table (``tq_codebook``), rounded to
fp32 exactly as the reference builds them; ``quantize`` / ``dequantize`` are thin device ops on
tensors the caller already holds on the GPU.
"""
from __future__ import annotations

import math

import torch

from . import _cabi


class Codebook:
    """Scalar quantization codebook for a rotated unit vector of dimension ``dim``."""

    def __init__(self, dim: int, bit_width: int, device="cuda"):
        assert 1 <= bit_width <= 4, f"Supported bit-widths: 1-4, got {bit_width}"
        self.dim = dim
        self.bit_width = bit_width
        self.num_levels = 1 << bit_width
        self.scale = 1.0 / math.sqrt(dim)
        cen, bnd = _cabi.codebook(dim, bit_width)
        self.centroids = cen.to(device)
        self.boundaries = bnd.to(device)

    @torch.no_grad()
    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Index of the nearest centroid (number of boundaries strictly below the value)."""
        return torch.bucketize(x, self.boundaries).to(torch.uint8)

    @torch.no_grad()
    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        return self.centroids[indices.long()]
