"""Head size 96 (padded to 128 by the rotation, turboquant/hadamard.py:66-68; same 80-byte slot):
cache write bit for bit, decode and bulk dequantization against the oracle, through the same
kernels as head size 128."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
from tests.gpu_util import DEV, assert_attention_close, signs_dev

pytestmark = pytest.mark.gpu
D = 96
SCALE = 1.0 / math.sqrt(D)


def _case(seed, lens, heads=(32, 8)):
    return synthetic.decode_case(seed=seed, seq_lens=lens, heads=heads, head_dim=D, dtype=torch.float16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_write_head96_bit_exact(oracle, golden, dtype):
    case = _case(5, [300, 17, 64])
    k, v = case.k.to(dtype), case.v.to(dtype)
    signs_np = golden["signs_seed42_d128"]
    want = np.full((2, case.num_blocks, 16, 8, 80), 0x33, np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), signs_np, case.slot_mapping.numpy(), D)
    cache = torch.full((2, case.num_blocks, 16, 8, 80), 0x33, dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, k.to(DEV), v.to(DEV), signs_dev(), case.slot_mapping.to(DEV), D)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(cache.cpu().numpy(), want)


def test_write_head96_matches_reference_fixture(golden, oracle):
    """The 96-wide quantizer rows of the reference fixture, written as K rows of one head."""
    rows = torch.from_numpy(golden["q_rows_d96"])
    n = rows.shape[0]
    cache = torch.zeros((2, (n + 15) // 16, 16, 1, 80), dtype=torch.uint8, device=DEV)
    k = rows.view(n, 1, D).to(DEV)
    _cabi.write_kv_cache(cache, k, k, torch.from_numpy(golden["signs_seed42_d96"]).to(DEV),
                         torch.arange(n, dtype=torch.int64, device=DEV), D)
    got = cache.cpu().numpy()[0].reshape(-1, 80)[:n]
    np.testing.assert_array_equal(got[:, :64], oracle.low_first_to_cache_order(golden["q_packed_d96"]))
    norms = got[:, 64:66].copy().view(np.float16).reshape(n)
    want = torch.from_numpy(golden["q_norms_d96"]).to(torch.float16).numpy()
    np.testing.assert_array_equal(norms.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("heads", [(32, 8), (8, 2), (32, 32)])
def test_decode_and_dequant_head96(oracle, golden, heads):
    lens = [700, 0, 33, 2049]
    case = _case(6, lens, heads)
    signs_np = golden["signs_seed42_d128"]
    cache = np.zeros((2, case.num_blocks, 16, heads[1], 80), np.uint8)
    oracle.write_kv_cache(cache, case.k.float().numpy(), case.v.float().numpy(), signs_np, case.slot_mapping.numpy(), D)
    want, want_lse = oracle.decode_paged(case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                                         signs_np, SCALE, return_lse=True)
    attn = TurboQuantPagedAttention(heads[0], D, SCALE, heads[1])
    cache_d = torch.from_numpy(cache).to(DEV)
    lse = torch.empty(len(lens), heads[0], dtype=torch.float32, device=DEV)
    out = attn.decode(case.q.to(DEV), cache_d, case.block_table.to(DEV), case.seq_lens.to(DEV), out_lse=lse)
    torch.cuda.synchronize()
    assert attn.status(len(lens), DEV) == 0 and out.shape == (len(lens), heads[0], D)
    assert_attention_close(out.float().cpu().numpy(), want, f"head 96, heads {heads}")
    ok = np.isfinite(want_lse)
    np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=3e-3)
    # bulk dequantization: fp32 bit for bit
    total = sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    k, v = attn.dequant_cached(cache_d, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, total, dtype=torch.float32)
    ks = []
    for b, n in enumerate(lens):
        t = np.arange(n)
        pages = case.block_table.numpy()[b, t // 16]
        ks.append(oracle.dequant_cache_rows(cache[0, pages, t % 16], signs_np, D))
    assert k.shape == (total, heads[1], D)
    np.testing.assert_array_equal(k.cpu().numpy(), np.concatenate(ks))


def test_wide_tile_and_causal_queries_head96(oracle, golden):
    """Head size 96 through the wide-tile kernel: 8 shared-KV queries and 5 causal ones."""
    lens = [700, 0, 33, 2049]
    heads = (32, 8)
    case = _case(8, lens, heads)
    signs_np = golden["signs_seed42_d128"]
    cache = np.zeros((2, case.num_blocks, 16, heads[1], 80), np.uint8)
    oracle.write_kv_cache(cache, case.k.float().numpy(), case.v.float().numpy(), signs_np, case.slot_mapping.numpy(), D)
    attn = TurboQuantPagedAttention(heads[0], D, SCALE, heads[1])
    cache_d, bt, sl = torch.from_numpy(cache).to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV)
    B = len(lens)
    for nq, causal in ((8, False), (5, True)):
        q = torch.randn(B, nq, heads[0], D, generator=torch.Generator().manual_seed(nq)).to(torch.float16)
        off = torch.arange(nq - 1, -1, -1, dtype=torch.int32).repeat(B) if causal else torch.zeros(B * nq, dtype=torch.int32)
        rep_len = (case.seq_lens.repeat_interleave(nq) - off).clamp(min=0)
        want = oracle.decode_paged(q.view(B * nq, heads[0], D).float().numpy(), cache,
                                   case.block_table.repeat_interleave(nq, dim=0).numpy(), rep_len.numpy(), signs_np, SCALE)
        out = (attn.decode_causal if causal else attn.decode_shared)(q.to(DEV), cache_d, bt, sl)
        torch.cuda.synchronize()
        assert attn.status(B, DEV, nq) == 0 and out.shape == (B, nq, heads[0], D)
        assert_attention_close(out.float().cpu().numpy().reshape(B * nq, heads[0], D), want, f"head 96, nq={nq}, causal={causal}")
