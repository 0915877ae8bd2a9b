"""Bulk dequantization of cached tokens (tq_dequant_paged) against the CPU oracle: fp32 output bit
for bit, fp16/bf16 output as its rounding; ragged lengths, an empty sequence, permuted pages, the
indptr form of the page table; and end to end: attention over the dequantized K/V equals the
decode kernel's answer."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from turboquant_b200.paged_attention import TurboQuantPagedAttention
from tests.gpu_util import DEV, assert_attention_close, oracle_cache, run_decode, signs_dev

pytestmark = pytest.mark.gpu


def _oracle_dense(oracle, cache, block_table, lens, signs_np):
    ks, vs = [], []
    for b, n in enumerate(lens):
        t = np.arange(n)
        pages = block_table[b, t // 16]
        ks.append(oracle.dequant_cache_rows(cache[0, pages, t % 16], signs_np, 128))
        vs.append(oracle.dequant_cache_rows(cache[1, pages, t % 16], signs_np, 128))
    return np.concatenate(ks), np.concatenate(vs)


@pytest.mark.parametrize("heads", [(32, 8), (8, 2), (4, 1)])
def test_dequant_paged_matches_oracle(oracle, golden, heads):
    lens = [37, 0, 512, 16, 1, 1000]
    case = synthetic.decode_case(seed=50 + heads[1], seq_lens=lens, heads=heads, dtype=torch.float16)
    signs_np = golden["signs_seed42_d128"]
    cache = oracle_cache(oracle, case, signs_np)
    want_k, want_v = _oracle_dense(oracle, cache, case.block_table.numpy(), lens, signs_np)
    total = sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    cache_d = torch.from_numpy(cache).to(DEV)
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        k = torch.full((total, heads[1], 128), float("nan"), dtype=dtype, device=DEV)
        v = torch.full_like(k, float("nan"))
        _cabi.dequant_paged(cache_d, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, signs_dev(), k, v)
        torch.cuda.synchronize()
        if dtype == torch.float32:
            assert np.array_equal(k.cpu().numpy(), want_k) and np.array_equal(v.cpu().numpy(), want_v)
        else:
            assert torch.equal(k.cpu(), torch.from_numpy(want_k).to(dtype))
            assert torch.equal(v.cpu(), torch.from_numpy(want_v).to(dtype))


def test_dequant_paged_indptr_and_stride(oracle, golden):
    lens = [100, 48, 7]
    case = synthetic.decode_case(seed=61, seq_lens=lens, dtype=torch.float16)
    signs_np = golden["signs_seed42_d128"]
    cache = oracle_cache(oracle, case, signs_np)
    want_k, want_v = _oracle_dense(oracle, cache, case.block_table.numpy(), lens, signs_np)
    bt = case.block_table.numpy()
    pages = [(n + 15) // 16 for n in lens]
    flat = np.concatenate([bt[b, :pages[b]] for b in range(len(lens))]).astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    total = sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    kv = torch.zeros(total, 2, 8, 128, dtype=torch.float32, device=DEV)   # K and V interleaved per token
    k, v = kv[:, 0], kv[:, 1]
    _cabi.dequant_paged(torch.from_numpy(cache).to(DEV), torch.from_numpy(flat).to(DEV), case.seq_lens.to(DEV), cu,
                        signs_dev(), k, v, page_indptr=torch.from_numpy(indptr).to(DEV), max_pages=max(pages))
    torch.cuda.synchronize()
    assert np.array_equal(k.cpu().numpy(), want_k) and np.array_equal(v.cpu().numpy(), want_v)


def test_attention_over_dequantized_cache_equals_decode(oracle, golden):
    """softmax(q K^T) V on the dequantized K/V (torch, fp32) against the decode kernel on the cache."""
    lens = [700, 33]
    case = synthetic.decode_case(seed=62, seq_lens=lens, dtype=torch.float16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    attn = TurboQuantPagedAttention(32, 128, 1 / math.sqrt(128), 8)
    cu = torch.tensor([0, 700, 733], dtype=torch.int32, device=DEV)
    k, v = attn.dequant_cached(cache, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, 733, dtype=torch.float32)
    out = run_decode(case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV)).float()
    for b, (s, e) in enumerate([(0, 700), (700, 733)]):
        q = case.q[b].float().to(DEV).view(8, 4, 128)                       # [kv head, group, d]
        sc = torch.einsum("hgd,thd->hgt", q, k[s:e]) / math.sqrt(128)
        ref = torch.einsum("hgt,thd->hgd", torch.softmax(sc, -1), v[s:e]).reshape(32, 128)
        assert_attention_close(out[b].cpu().numpy(), ref.cpu().numpy(), f"sequence {b}")


def test_dequant_paged_rejects_bad_arguments():
    cache = torch.zeros(2, 4, 16, 8, 80, dtype=torch.uint8, device=DEV)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    sl = torch.ones(1, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    k = torch.zeros(1, 8, 16, dtype=torch.float32, device=DEV)
    with pytest.raises(_cabi.TurboQuantError, match="head_dim"):
        _cabi.dequant_paged(cache, bt, sl, cu, signs_dev(), k, torch.zeros_like(k))
