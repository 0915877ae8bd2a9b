"""The allocation-free decode entry point (tq_decode_paged_static), through the C ABI.

It serves callers that cannot create or pass a workspace (a plugin inside an engine whose memory
pool is fully assigned, or a path where cudaMalloc is forbidden): the split-KV scratch is a fixed
array inside the library.  Its output must equal that of the ordinary entry point, which gets a
caller-allocated workspace, on two calls in a row (the array keeps the previous call's contents),
and a request beyond the array's size must be refused with a clear message.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCALE = 1.0 / math.sqrt(128)


def _case(seed, lens):
    case = synthetic.decode_case(seed=seed, seq_lens=lens, dtype=torch.bfloat16)
    signs = synthetic.make_signs(128, 42).to(DEV)
    cache = torch.zeros((2, case.num_blocks, 16, 8, 80), dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, case.k.to(DEV), case.v.to(DEV), signs, case.slot_mapping.to(DEV), 128)
    return case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV), signs


def _reference(q, cache, bt, sl, signs):
    ws = torch.zeros(_cabi.decode_workspace_bytes(q.shape[0], 32, 8), dtype=torch.uint8, device=DEV)
    out = torch.empty(q.shape, dtype=torch.float32, device=DEV)
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device=DEV)
    _cabi.decode_paged(q, cache, bt, sl, signs, SCALE, ws, out, out_lse=lse)
    torch.cuda.synchronize()
    return out.cpu().numpy(), lse.cpu().numpy()


def test_static_scratch_matches_workspace_entry_point_twice():
    assert _cabi.decode_workspace_bytes(4, 32, 8) <= _cabi.STATIC_SCRATCH_BYTES
    first = _case(71, [700, 33, 2049, 1])
    second = _case(72, [64, 5000])          # different shapes: stale contents of the array must not leak
    for q, cache, bt, sl, signs in (first, second, first):
        want, want_lse = _reference(q, cache, bt, sl, signs)
        out = torch.empty(q.shape, dtype=torch.float32, device=DEV)
        lse = torch.empty(q.shape[:2], dtype=torch.float32, device=DEV)
        free_before = torch.cuda.mem_get_info()[0]
        _cabi.decode_paged_static(q, cache, bt, sl, signs, SCALE, out, out_lse=lse)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before      # nothing was allocated on the device
        # same kernels, same split plan: the tolerance of the split-invariance tests (3e-4) is ample
        np.testing.assert_allclose(out.cpu().numpy(), want, atol=3e-4, rtol=1e-3)
        np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=1e-4)


def test_request_beyond_the_static_scratch_is_refused():
    q, cache, bt, sl, signs = _case(73, [40])
    big = 4096                                # scratch need grows with the batch
    qb = q.expand(big, 32, 128).contiguous()
    out = torch.empty_like(qb)
    with pytest.raises(_cabi.TurboQuantError, match="built-in scratch"):
        _cabi.decode_paged_static(qb, cache, bt.expand(big, -1).contiguous(), sl.expand(big).contiguous(),
                                  signs, SCALE, out)
