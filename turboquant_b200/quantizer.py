"""TurboQuantMSE with the reference's interface (turboquant/quantizer.py:60-106), computed by
the library's flat quantizer kernels; codes and norms are bit-identical to the reference's
torch CPU results."""
from __future__ import annotations

import torch

from . import _cabi
from .codebook import Codebook
from .hadamard import RandomHadamardRotation


class TurboQuantMSE:
    """norm -> normalize -> randomized Hadamard rotation -> Lloyd-Max code -> bit pack."""

    def __init__(self, dim: int, bit_width: int, device="cuda", seed: int = 42):
        self.dim = dim
        self.bit_width = bit_width
        self.device = device
        self.rotation = RandomHadamardRotation(dim, device=device, seed=seed)
        self.codebook = Codebook(self.rotation.padded_dim, bit_width, device=device)

    @torch.no_grad()
    def quantize(self, x: torch.Tensor):
        """x [..., d] -> (packed uint8 [..., padded*bits/8] in the low-first order of the
        reference's ``_pack_bits``, norms fp32 [...])."""
        return _cabi.quantize_flat(x, self.rotation.signs, self.bit_width, cache_order=False)

    @torch.no_grad()
    def quantize_cache_order(self, x: torch.Tensor):
        """Same codes packed the way the paged cache stores them (even dim in the high nibble)."""
        return _cabi.quantize_flat(x, self.rotation.signs, self.bit_width, cache_order=True)

    @torch.no_grad()
    def dequantize(self, packed: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        return _cabi.dequantize_flat(packed, norms, self.rotation.signs, self.dim, self.bit_width)
