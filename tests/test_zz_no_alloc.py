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
        # Nothing may be allocated on the device.  Free memory as the driver reports it can also move
        # when another process uses the GPU, so a difference is re-checked before it counts.
        for attempt in range(3):
            free_before = torch.cuda.mem_get_info()[0]
            _cabi.decode_paged_static(q, cache, bt, sl, signs, SCALE, out, out_lse=lse)
            torch.cuda.synchronize()
            if torch.cuda.mem_get_info()[0] == free_before:
                break
        else:
            raise AssertionError("free device memory changed across three calls in a row")
        assert _cabi.decode_static_status() == 0                # every block wrote its partials
        # same kernels, same split plan: the tolerance of the split-invariance tests (3e-4) is ample
        np.testing.assert_allclose(out.cpu().numpy(), want, atol=3e-4, rtol=1e-3)
        np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=1e-4)


def test_documented_limits_of_the_static_scratch():
    """The numbers the header and the integration notes give for one block per SM on 148 SMs."""
    fits = _cabi.decode_workspace_bytes(105, 32, 8, 128, 148)
    over = _cabi.decode_workspace_bytes(106, 32, 8, 128, 148)
    assert fits <= _cabi.STATIC_SCRATCH_BYTES < over
    assert _cabi.decode_workspace_bytes(1, 32, 4, 128, 148) > _cabi.STATIC_SCRATCH_BYTES   # 32 q / 4 kv heads never fit
    q, cache, bt, sl, signs = _case(74, [40])
    with pytest.raises(_cabi.TurboQuantError, match="1, 2, 4, 8 or 16"):
        c32 = torch.zeros((2, 4, 16, 32, 80), dtype=torch.uint8, device=DEV)
        _cabi.decode_paged_static(q, c32, bt, sl, signs, SCALE, torch.empty_like(q))


def test_request_beyond_the_static_scratch_is_refused():
    q, cache, bt, sl, signs = _case(73, [40])
    big = 4096                                # scratch need grows with the batch
    qb = q.expand(big, 32, 128).contiguous()
    out = torch.empty_like(qb)
    with pytest.raises(_cabi.TurboQuantError, match="built-in scratch"):
        _cabi.decode_paged_static(qb, cache, bt.expand(big, -1).contiguous(), sl.expand(big).contiguous(),
                                  signs, SCALE, out)
