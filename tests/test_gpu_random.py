"""Seeded random sweeps of shapes through the C ABI against the oracle: the cache write (token
counts, head counts incl. non-powers of two, dtypes, padded token strides, int32 / int64 slots,
skipped slots, magnitudes) bit for bit, and the decode (batch sizes, lengths incl. empty and
one-token sequences, head geometries, dtypes, block counts, both page-table forms, queries that
share a sequence) within the attention tolerance."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from tests.gpu_util import DEV, assert_attention_close, signs_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", range(12))
def test_random_cache_writes_bit_exact(oracle, golden, case):
    rng = np.random.default_rng(1000 + case)
    T = int(rng.integers(1, 700))
    H = int(rng.choice([1, 2, 3, 4, 5, 8]))
    dtype = [torch.float32, torch.float16, torch.bfloat16][case % 3]
    pad = int(rng.choice([0, 8, 64]))                            # extra elements per token row (multiple of 8)
    g = torch.Generator().manual_seed(2000 + case)
    scale = float(10.0 ** rng.uniform(-3, 3))
    kbuf = (torch.randn(T, H * 128 + pad, generator=g) * scale).to(dtype)
    vbuf = (torch.randn(T, H * 128 + pad, generator=g) * scale).to(dtype)
    k = kbuf[:, : H * 128].view(T, H, 128)
    v = vbuf[:, : H * 128].view(T, H, 128)
    nb = (T + 15) // 16 + 3
    slots = torch.from_numpy(rng.permutation(nb * 16)[:T].astype(np.int64))
    slots[torch.from_numpy(rng.random(T) < 0.1)] = -1
    if case % 2:
        slots = slots.to(torch.int32)
    signs_np = golden["signs_seed42_d128"]
    want = np.full((2, nb, 16, H, 80), 0x5A, np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), signs_np, slots.numpy(), 128)
    cache = torch.full((2, nb, 16, H, 80), 0x5A, dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, kbuf.to(DEV)[:, : H * 128].view(T, H, 128), vbuf.to(DEV)[:, : H * 128].view(T, H, 128),
                         signs_dev(), slots.to(DEV), 128)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(cache.cpu().numpy(), want)


@pytest.mark.parametrize("case", range(10))
def test_random_decodes_match_oracle(oracle, golden, case):
    rng = np.random.default_rng(3000 + case)
    hq, hkv = [(32, 8), (16, 4), (8, 2), (4, 1), (8, 8), (64, 8), (24, 8), (12, 4), (2, 2), (40, 8)][case]
    B = int(rng.integers(1, 13))
    lens = [int(x) for x in rng.choice([0, 1, 15, 16, 17, 100, 333, 1024, 2500], size=B)]
    if sum(lens) == 0:
        lens[0] = 50
    q_dtype = [torch.float16, torch.bfloat16, torch.float32][case % 3]
    case_ = synthetic.decode_case(seed=4000 + case, seq_lens=lens, heads=(hq, hkv), dtype=torch.float16)
    signs_np = golden["signs_seed42_d128"]
    cache = np.zeros((2, case_.num_blocks, 16, hkv, 80), np.uint8)
    oracle.write_kv_cache(cache, case_.k.float().numpy(), case_.v.float().numpy(), signs_np,
                          case_.slot_mapping.numpy(), 128)
    q = case_.q.to(q_dtype)
    scale = float(rng.choice([1 / math.sqrt(128), 0.05, 0.2]))
    want, want_lse = oracle.decode_paged(q.float().numpy(), cache, case_.block_table.numpy(), case_.seq_lens.numpy(),
                                         signs_np, scale, return_lse=True)
    ctas = int(rng.choice([0, 1, 3, 37, 148]))
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, hq, hkv, 128, ctas), dtype=torch.uint8, device=DEV)
    out = torch.full((B, hq, 128), float("nan"), dtype=q_dtype, device=DEV)
    lse = torch.empty(B, hq, dtype=torch.float32, device=DEV)
    cache_d = torch.from_numpy(cache).to(DEV)
    if case % 2:   # CSR form of the page table
        bt = case_.block_table.numpy()
        pages = [(n + 15) // 16 for n in lens]
        flat = np.concatenate([bt[b, :pages[b]] for b in range(B)] + [np.zeros(1, np.int32)]).astype(np.int32)
        indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
        _cabi.decode_paged(q.to(DEV), cache_d, torch.from_numpy(flat).to(DEV), case_.seq_lens.to(DEV), signs_dev(),
                           scale, ws, out, page_indptr=torch.from_numpy(indptr).to(DEV), out_lse=lse, num_ctas=ctas,
                           max_pages=max(max(pages), 1))
    else:
        _cabi.decode_paged(q.to(DEV), cache_d, case_.block_table.to(DEV), case_.seq_lens.to(DEV), signs_dev(), scale,
                           ws, out, out_lse=lse, num_ctas=ctas)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    got = out.float().cpu().numpy()
    assert_attention_close(got, want, f"case {case}: heads {hq}/{hkv}, lens {lens}, ctas {ctas}")
    for b, n in enumerate(lens):
        if n == 0:
            assert (got[b] == 0).all()
    ok = np.isfinite(want_lse)
    np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=3e-3)
