"""Fast Walsh-Hadamard transform and the seeded randomized rotation, with the reference's
interface (turboquant/hadamard.py:14-78), computed by the library's FWHT kernel (``tq_fwht``)."""
from __future__ import annotations

import torch

from . import _cabi
from .synthetic import make_signs


def next_power_of_2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


@torch.no_grad()
def fwht(x: torch.Tensor) -> torch.Tensor:
    """Normalized FWHT along the last dimension (a power of two up to 256): (1/sqrt(d)) H x."""
    d = x.shape[-1]
    assert d > 0 and (d & (d - 1)) == 0, f"Last dim must be power of 2, got {d}"
    return _cabi.fwht(x, d, d).to(x.dtype)


class RandomHadamardRotation:
    """y = FWHT(signs * pad(x));  x = unpad(signs * FWHT(y)).  Signs from a CPU generator seeded
    with ``seed`` (sign(randn), 0 -> +1), as in the reference."""

    def __init__(self, dim: int, device="cuda", seed: int = 42):
        self.orig_dim = dim
        self.padded_dim = next_power_of_2(dim)
        self.signs = make_signs(self.padded_dim, seed).to(device)

    @torch.no_grad()
    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return _cabi.fwht(x, self.padded_dim, self.padded_dim, pre_signs=self.signs).to(x.dtype)

    @torch.no_grad()
    def inverse_rotate(self, y: torch.Tensor) -> torch.Tensor:
        return _cabi.fwht(y, self.padded_dim, self.orig_dim, post_signs=self.signs).to(y.dtype)
