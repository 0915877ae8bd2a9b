"""The oracle against the torch that is installed on this machine.

The reference quantizer is a handful of torch calls (turboquant/quantizer.py:77-91: ``norm``,
``clamp``, a division, the signs, the butterfly transform of turboquant/hadamard.py:21-42 and
``bucketize``); how ``Tensor.norm`` orders its additions is a property of the torch build and of the
CPU it runs on, not of the reference.  The fixtures pin one build; this test re-derives the
quantizer from live torch on whatever host runs it (it is also collected under ``-m gpu`` so that
the GPU box's host is covered) and fails loudly if the oracle's fixed evaluation order no longer
reproduces it bit for bit."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import synthetic


def _torch_quantize(x: torch.Tensor, signs: torch.Tensor, boundaries: torch.Tensor):
    norms = x.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    y = (x / norms) * signs
    d = y.shape[-1]
    h = 1
    while h < d:                                  # butterflies, stage order h = 1, 2, 4, ...
        y = y.view(-1, d // (2 * h), 2, h)
        y = torch.stack((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), dim=2).reshape(-1, d)
        h *= 2
    y = y * (1.0 / math.sqrt(d))
    idx = torch.bucketize(y, boundaries)
    packed = (idx[:, 0::2] | idx[:, 1::2] << 4).to(torch.uint8)       # first index in the low nibble (quantizer.py:17-35)
    return packed, norms.squeeze(-1)


def _check(oracle):
    g = torch.Generator().manual_seed(1234)
    rows = torch.randn(4096, 128, generator=g)
    rows[::7] = rows[::7].to(torch.bfloat16).float()          # bf16-sourced rows
    rows[::11, 5] *= 20.0                                       # an outlier channel
    rows[100] = 0.0
    rows[101] = 1e-9
    rows[102, 3] = 1e20
    signs = synthetic.make_signs(128, 42)
    _, bnd = oracle.codebook(128, 4)
    want_p, want_n = _torch_quantize(rows, signs, torch.from_numpy(bnd))
    got_p, got_n = oracle.quantize_flat(rows.numpy(), signs.numpy(), 4)
    np.testing.assert_array_equal(got_n.view(np.uint32), want_n.numpy().view(np.uint32))
    np.testing.assert_array_equal(got_p, want_p.numpy())


def test_oracle_matches_live_torch_on_this_host(oracle):
    _check(oracle)


@pytest.mark.gpu
def test_oracle_matches_live_torch_on_the_gpu_host(oracle):
    _check(oracle)
