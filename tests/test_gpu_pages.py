"""Offload / restore of packed pages: the round trip restores every information byte of the moved
pages (into other page ids as well), touches nothing else, and a decode over the restored cache
equals the decode over the original."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from turboquant_b200.paged_attention import TurboQuantPagedAttention
from tests.gpu_util import DEV, oracle_cache, run_decode

pytestmark = pytest.mark.gpu


def test_gather_layout_and_round_trip():
    g = torch.Generator().manual_seed(9)
    cache = torch.randint(0, 256, (2, 40, 16, 8, 80), dtype=torch.uint8, generator=g)
    ids = torch.tensor([7, 0, 39, 12, 13], dtype=torch.int32)
    cache_d = cache.to(DEV)
    packed = torch.zeros(_cabi.pages_packed_bytes(5, 16, 8), dtype=torch.uint8, device=DEV)
    _cabi.pages_gather(cache_d, ids.to(DEV), packed)
    want = cache[:, ids.long()][..., :68].permute(1, 0, 2, 3, 4).contiguous()      # [n, 2, 16, 8, 68]
    assert torch.equal(packed.cpu().view(5, 2, 16, 8, 68), want)
    # restore into other pages of a cache full of 0xAB: payload restored, pad and other pages untouched
    dst = torch.full_like(cache_d, 0xAB)
    new_ids = torch.tensor([1, 2, 3, 30, 31], dtype=torch.int32, device=DEV)
    _cabi.pages_scatter(dst, new_ids, packed)
    out = dst.cpu()
    assert torch.equal(out[:, new_ids.cpu().long()][..., :68], cache[:, ids.long()][..., :68])
    assert (out[:, new_ids.cpu().long()][..., 68:] == 0xAB).all()
    rest = torch.ones(40, dtype=torch.bool)
    rest[new_ids.cpu().long()] = False
    assert (out[:, rest] == 0xAB).all()


def test_offload_restore_then_decode(oracle, golden):
    lens = [300, 1000]
    case = synthetic.decode_case(seed=71, seq_lens=lens, dtype=torch.float16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    attn = TurboQuantPagedAttention(32, 128, 1 / math.sqrt(128), 8)
    want = run_decode(case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV))
    # offload the pages of sequence 1, wipe them, restore them into fresh page ids
    pages1 = case.block_table[1, : (1000 + 15) // 16].to(DEV)
    host = attn.offload_pages(cache, pages1)
    torch.cuda.synchronize()
    assert host.is_pinned() and host.numel() == pages1.numel() * 2 * 16 * 8 * 68
    cache[:, pages1.long()] = 0
    bigger = torch.zeros(2, cache.shape[1] + 80, 16, 8, 80, dtype=torch.uint8, device=DEV)
    bigger[:, : cache.shape[1]] = cache
    fresh = torch.arange(cache.shape[1], cache.shape[1] + pages1.numel(), dtype=torch.int32, device=DEV)
    attn.restore_pages(bigger, fresh, host)
    bt = case.block_table.clone().to(DEV)
    bt[1, : pages1.numel()] = fresh
    got = run_decode(case.q.to(DEV), bigger, bt, case.seq_lens.to(DEV))
    assert torch.equal(got, want)


def test_pages_reject_small_buffer():
    cache = torch.zeros(2, 4, 16, 8, 80, dtype=torch.uint8, device=DEV)
    ids = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(_cabi.TurboQuantError, match="too small"):
        _cabi.pages_gather(cache, ids, torch.zeros(100, dtype=torch.uint8, device=DEV))
