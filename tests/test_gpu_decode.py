"""Paged decode-attention parity on the GPU, through the C ABI: against the fixtures made by
the reference's dequant-attention path, against the CPU oracle, and through size-independent
properties (split invariance, partial + merge == full) at the benchmark's full size."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from tests.gpu_util import DEV, assert_attention_close, fill_cache_gpu, oracle_cache, run_decode, signs_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128)


def test_golden_ragged_batch(golden):
    cache = torch.from_numpy(golden["att_cache"]).to(DEV)
    q = torch.from_numpy(golden["att_q"]).to(DEV)
    out, lse = run_decode(q, cache, torch.from_numpy(golden["att_block_table"]).to(DEV),
                          torch.from_numpy(golden["att_seq_lens"]).to(DEV), want_lse=True)
    assert_attention_close(out.float().cpu().numpy(), golden["att_out"], "golden ragged batch")
    np.testing.assert_allclose(lse.cpu().numpy(), golden["att_lse"], atol=2e-3)


def test_config0_vs_reference_output(golden, oracle):
    c0 = synthetic.decode_case(seed=0, seq_lens=[1024], dtype=torch.float16, permute_pages=False)
    cache = oracle_cache(oracle, c0, golden["signs_seed42_d128"])
    out, lse = run_decode(c0.q.to(DEV), torch.from_numpy(cache).to(DEV), c0.block_table.to(DEV),
                          c0.seq_lens.to(DEV), want_lse=True)
    assert_attention_close(out.float().cpu().numpy(), golden["cfg0_out"], "config 0", strict=True)
    np.testing.assert_allclose(lse.cpu().numpy(), golden["cfg0_lse"], atol=2e-3)


def test_write_then_decode_end_to_end(golden):
    """Cache produced by the CUDA write kernel, decoded by the CUDA decode kernel (config 0)."""
    c0 = synthetic.decode_case(seed=0, seq_lens=[1024], dtype=torch.float16, permute_pages=False)
    cache = torch.zeros((2, c0.num_blocks, 16, 8, 80), dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, c0.k.to(DEV), c0.v.to(DEV), signs_dev(), c0.slot_mapping.to(DEV), 128)
    out = run_decode(c0.q.to(DEV), cache, c0.block_table.to(DEV), c0.seq_lens.to(DEV))
    assert_attention_close(out.float().cpu().numpy(), golden["cfg0_out"], "write+decode config 0")


@pytest.mark.parametrize("q_dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32),
                                               (torch.float32, torch.float16)])
def test_mixed_lengths_vs_oracle(oracle, golden, q_dtype, out_dtype):
    lens = [1, 15, 16, 17, 700, 2049, 0, 333]
    case = synthetic.decode_case(seed=21, seq_lens=lens, dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    q = case.q.to(q_dtype)
    want, want_lse = oracle.decode_paged(q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                                         golden["signs_seed42_d128"], SCALE, return_lse=True)
    for ctas in (0, 1, 5):
        out, lse = run_decode(q.to(DEV), torch.from_numpy(cache).to(DEV), case.block_table.to(DEV),
                              case.seq_lens.to(DEV), out_dtype=out_dtype, num_ctas=ctas, want_lse=True)
        got = out.float().cpu().numpy()
        assert_attention_close(got, want, f"mixed lengths, ctas={ctas}")
        assert (got[6] == 0).all()                                   # empty sequence -> zeros
        ok = np.isfinite(want_lse)
        np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=2e-3)
        assert np.isneginf(lse.cpu().numpy()[~ok]).all()


@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 4), (16, 2), (8, 1), (8, 8), (64, 8), (4, 4), (16, 16), (32, 16),
                                    (64, 16), (32, 32), (40, 40), (24, 12), (40, 20), (64, 32)])
def test_head_geometries(oracle, golden, hq, hkv):
    case = synthetic.decode_case(seed=30 + hq + hkv, seq_lens=[300, 45, 1000], dtype=torch.float16, heads=(hq, hkv))
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    want = oracle.decode_paged(case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    for ctas in (0, 3):
        out = run_decode(case.q.to(DEV), torch.from_numpy(cache).to(DEV), case.block_table.to(DEV),
                         case.seq_lens.to(DEV), num_ctas=ctas)
        assert_attention_close(out.float().cpu().numpy(), want, f"hq={hq} hkv={hkv} ctas={ctas}")


def test_peaked_softmax_and_scale(oracle, golden):
    """A query aligned with one key (one token dominates) and a non-default softmax scale."""
    case = synthetic.decode_case(seed=41, seq_lens=[513, 64], dtype=torch.float16)
    case.q[0] = case.k[100].repeat_interleave(4, dim=0) * 2.0
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    for scale in (SCALE, 0.25):
        want = oracle.decode_paged(case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                                   golden["signs_seed42_d128"], scale)
        out = run_decode(case.q.to(DEV), torch.from_numpy(cache).to(DEV), case.block_table.to(DEV),
                         case.seq_lens.to(DEV), sm_scale=scale, out_dtype=torch.float32)
        got = out.cpu().numpy()
        # outputs are O(1) here; fp16 operand rounding scales with magnitude, so use the mixed bar
        assert np.abs(got - want).max() <= 2e-3 + 1e-2 * np.abs(want).max()
        assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-2


def test_csr_page_table(oracle, golden):
    case = synthetic.decode_case(seed=50, seq_lens=[100, 33, 260], dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    want = oracle.decode_paged(case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    pages = [(int(n) + 15) // 16 for n in case.seq_lens]
    indptr = torch.tensor([0] + list(np.cumsum(pages)), dtype=torch.int32)
    indices = torch.cat([case.block_table[b, :p] for b, p in enumerate(pages)]).to(torch.int32)
    out = run_decode(case.q.to(DEV), torch.from_numpy(cache).to(DEV), indices.to(DEV), case.seq_lens.to(DEV),
                     page_indptr=indptr.to(DEV))
    assert_attention_close(out.float().cpu().numpy(), want, "CSR page table")


def test_partial_plus_merge_equals_full(oracle, golden):
    """KV-axis split (the multi-GPU contract): per-window rotated partials + LSE merge == full."""
    case = synthetic.decode_case(seed=60, seq_lens=[1500, 90], dtype=torch.bfloat16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    q, bt, sl = case.q.to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV)
    full = run_decode(q, cache, bt, sl, out_dtype=torch.float32)
    ws = torch.zeros(_cabi.decode_workspace_bytes(2, 32, 8), dtype=torch.uint8, device=DEV)
    windows = [(0, 512), (512, 1024), (1024, -1), (2048, -1)]          # the last one is empty
    po = torch.empty(len(windows), 2, 32, 128, dtype=torch.float32, device=DEV)
    pl = torch.empty(len(windows), 2, 32, dtype=torch.float32, device=DEV)
    for i, (a, b) in enumerate(windows):
        _cabi.decode_paged_partial(q, cache, bt, sl, signs_dev(), SCALE, ws, po[i], pl[i], kv_begin=a, kv_end=b)
    assert torch.isneginf(pl[3]).all() and torch.isneginf(pl[1, 1]).all()
    out = torch.empty(2, 32, 128, dtype=torch.float32, device=DEV)
    lse = torch.empty(2, 32, dtype=torch.float32, device=DEV)
    _cabi.merge_rotated(po, pl, signs_dev(), out, lse)
    torch.cuda.synchronize()
    # different cuts round P to fp16 against different running maxima: agreement to ~1e-4
    np.testing.assert_allclose(out.cpu().numpy(), full.cpu().numpy(), atol=3e-4, rtol=1e-3)
    want, want_lse = oracle.decode_paged(case.q.float().numpy(), cache.cpu().numpy(), case.block_table.numpy(),
                                         case.seq_lens.numpy(), golden["signs_seed42_d128"], SCALE, return_lse=True)
    assert_attention_close(out.cpu().numpy(), want, "merged windows")
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=2e-3)


def test_merge_rotated_matches_oracle_merge(oracle):
    gen = torch.Generator().manual_seed(3)
    po = torch.randn(5, 7, 128, generator=gen)
    pl = torch.randn(5, 7, generator=gen) * 3
    pl[2, 3] = -math.inf
    pl[:, 5] = -math.inf
    signs = synthetic.make_signs()
    out = torch.empty(7, 128, dtype=torch.float32, device=DEV)
    lse = torch.empty(7, dtype=torch.float32, device=DEV)
    _cabi.merge_rotated(po.to(DEV), pl.to(DEV), signs.to(DEV), out, lse)
    merged, mlse = oracle.merge_partials(po.numpy(), pl.numpy() * math.log(2.0))   # oracle is natural-log
    want = np.stack([oracle.fwht(merged[r]) * signs.numpy() for r in range(7)])
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=1e-5)
    ok = np.isfinite(mlse)
    np.testing.assert_allclose(lse.cpu().numpy()[ok], mlse[ok], atol=1e-5)
    assert (out.cpu().numpy()[5] == 0).all()


def test_config1_full_size_properties():
    """Batch 8 x 32768 tokens (one layer of the benchmark): the result must not depend on how the
    KV range is cut (296 vs 37 vs 8 thread blocks), and one sequence decoded alone must equal its
    row in the batch."""
    B, L = 8, 32768
    gen = torch.Generator().manual_seed(1)
    nb = B * L // 16
    cache = torch.zeros((2, nb, 16, 8, 80), dtype=torch.uint8, device=DEV)
    perm = torch.randperm(nb, generator=gen)
    bt = perm.view(B, L // 16).to(torch.int32).to(DEV)
    signs = signs_dev()
    for b in range(B):                                              # fill with the CUDA write kernel
        k = torch.randn(L, 8, 128, generator=gen).to(torch.bfloat16).to(DEV)
        v = torch.randn(L, 8, 128, generator=gen).to(torch.bfloat16).to(DEV)
        t = torch.arange(L, device=DEV)
        slots = bt[b].long()[t // 16] * 16 + t % 16
        _cabi.write_kv_cache(cache, k, v, signs, slots, 128)
    q = torch.randn(B, 32, 128, generator=gen).to(torch.bfloat16).to(DEV)
    sl = torch.full((B,), L, dtype=torch.int32, device=DEV)
    ref = run_decode(q, cache, bt, sl, out_dtype=torch.float32, num_ctas=296).cpu().numpy()
    assert np.isfinite(ref).all() and np.abs(ref).max() > 1e-3
    for ctas in (37, 8):
        out = run_decode(q, cache, bt, sl, out_dtype=torch.float32, num_ctas=ctas).cpu().numpy()
        assert np.abs(out - ref).max() <= 2e-4
    one = run_decode(q[3:4], cache, bt[3:4], sl[3:4], out_dtype=torch.float32).cpu().numpy()
    assert np.abs(one[0] - ref[3]).max() <= 2e-4
    # shorter length on a page boundary and off it: later tokens must not leak in
    sl2 = sl.clone()
    sl2[0] = 20000
    sl2[1] = 12345
    out2 = run_decode(q, cache, bt, sl2, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(out2[2:] - ref[2:]).max() <= 2e-4
    assert np.abs(out2[0] - ref[0]).max() > 1e-4


def test_config1_full_size_vs_oracle(oracle, golden):
    """One full layer of the benchmark's workload (batch 8 x 32768 tokens, bf16 queries and
    outputs, pages permuted) against the dequant-attention oracle run over the same bytes; the
    strict bar (max-abs 2e-3 and relative 1e-2) is asserted, not only the mixed one."""
    B, L = 8, 32768
    gen = torch.Generator(device=DEV)
    gen.manual_seed(1)
    nb = B * L // 16
    cache = torch.zeros((2, nb, 16, 8, 80), dtype=torch.uint8, device=DEV)
    bt = torch.randperm(nb, generator=torch.Generator().manual_seed(1)).view(B, L // 16).to(torch.int32).to(DEV)
    for b in range(B):
        fill_cache_gpu(cache, bt[b], L, gen)
    q = torch.randn(B, 32, 128, generator=gen, device=DEV).to(torch.bfloat16)
    sl = torch.full((B,), L, dtype=torch.int32, device=DEV)
    out, lse = run_decode(q, cache, bt, sl, out_dtype=torch.bfloat16, want_lse=True)
    want, want_lse = oracle.decode_paged_parallel(q.float().cpu().numpy(), cache.cpu().numpy(), bt.cpu().numpy(),
                                                  sl.cpu().numpy(), golden["signs_seed42_d128"], SCALE, return_lse=True)
    max_abs, rel = assert_attention_close(out.float().cpu().numpy(), want, "config 1, one full layer", strict=True)
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=2e-3)
    print(f"config 1 full size: max-abs {max_abs:.3e}, relative {rel:.3e}")


def test_config3_full_size_vs_oracle(oracle, golden):
    """The mixed-length config at its real size: 64 sequences, lengths log-uniform in
    [512, 131072] (seed 3), one layer, random block table, against the oracle."""
    lens = synthetic.mixed_lengths(seed=3, n=64)
    bt_cpu, _, nb = synthetic.paged_layout(lens, seed=3)
    bt = bt_cpu.to(DEV)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(3)
    cache = torch.zeros((2, nb, 16, 8, 80), dtype=torch.uint8, device=DEV)
    for b, n in enumerate(lens):
        fill_cache_gpu(cache, bt[b], n, gen)
    q = torch.randn(len(lens), 32, 128, generator=gen, device=DEV).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out, lse = run_decode(q, cache, bt, sl, out_dtype=torch.bfloat16, want_lse=True)
    want, want_lse = oracle.decode_paged_parallel(q.float().cpu().numpy(), cache.cpu().numpy(), bt_cpu.numpy(),
                                                  sl.cpu().numpy(), golden["signs_seed42_d128"], SCALE, return_lse=True)
    max_abs, rel = assert_attention_close(out.float().cpu().numpy(), want, "config 3, 64 mixed lengths", strict=True)
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=2e-3)
    print(f"config 3 full size: {sum(lens)} tokens, max-abs {max_abs:.3e}, relative {rel:.3e}")


def test_config4_full_size_vs_oracle(oracle, golden):
    """One sequence of 1,048,576 tokens with 8 decode queries that share its KV
    (tq_decode_paged_multi) against the oracle: the oracle sees the 8 queries as 32 query heads
    per KV head of one batch row, so it too dequantizes every token once."""
    total, nq = 1_048_576, 8
    pages = total // 16
    gen = torch.Generator(device=DEV)
    gen.manual_seed(4)
    bt_row = torch.randperm(pages, generator=torch.Generator().manual_seed(4)).to(torch.int32).to(DEV)
    cache = torch.zeros((2, pages, 16, 8, 80), dtype=torch.uint8, device=DEV)
    fill_cache_gpu(cache, bt_row, total, gen)
    q = torch.randn(nq, 32, 128, generator=gen, device=DEV).to(torch.bfloat16)
    share = _cabi.decode_max_queries_per_seq(32, 8)
    rows = nq // share
    qm = q.view(rows, share, 32, 128).contiguous()
    bt = bt_row.unsqueeze(0).expand(rows, -1).contiguous()
    sl = torch.full((rows,), total, dtype=torch.int32, device=DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(rows, share * 32, 8), dtype=torch.uint8, device=DEV)
    out = torch.empty_like(qm)
    lse = torch.empty(rows, share, 32, dtype=torch.float32, device=DEV)
    _cabi.decode_paged_multi(qm, cache, bt, sl, signs_dev(), SCALE, ws, out, out_lse=lse)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    # oracle: one batch row with 8 x 4 query heads per KV head; virtual head = kv * 32 + query * 4 + g
    qv = q.float().cpu().numpy().reshape(nq, 8, 4, 128).transpose(1, 0, 2, 3).reshape(1, 256, 128)
    want, want_lse = oracle.decode_paged_parallel(qv, cache.cpu().numpy(), bt_row.cpu().numpy()[None],
                                                  np.array([total], np.int32), golden["signs_seed42_d128"], SCALE,
                                                  chunk_tokens=16384, return_lse=True)
    want = want.reshape(8, nq, 4, 128).transpose(1, 0, 2, 3).reshape(nq, 32, 128)
    want_lse = want_lse.reshape(8, nq, 4).transpose(1, 0, 2).reshape(nq, 32)
    max_abs, rel = assert_attention_close(out.float().cpu().numpy().reshape(nq, 32, 128), want,
                                          "config 4, 1M tokens x 8 queries", strict=True)
    np.testing.assert_allclose(lse.cpu().numpy().reshape(nq, 32), want_lse, atol=2e-3)
    print(f"config 4 full size: max-abs {max_abs:.3e}, relative {rel:.3e}")


# the last five go through the wide-tile (tensor-memory) kernel: 9 to 32 query columns per KV head
@pytest.mark.parametrize("nq,hq,hkv", [(2, 32, 8), (8, 8, 8), (3, 8, 4), (4, 4, 2), (1, 32, 8),
                                       (8, 32, 8), (3, 32, 8), (5, 8, 4), (16, 4, 2), (9, 16, 16)])
def test_shared_kv_queries_match_repeated_rows(oracle, golden, nq, hq, hkv):
    """Several queries per sequence (tq_decode_paged_multi) against (a) the oracle with each query
    as its own batch row and (b) tq_decode_paged on the same repeated rows."""
    lens = [40, 0, 1000, 16, 2100]
    B = len(lens)
    case = synthetic.decode_case(seed=77 + nq, seq_lens=lens, heads=(hq, hkv), dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, nq, hq, 128, generator=g).to(torch.float16)
    rep_bt = case.block_table.repeat_interleave(nq, dim=0)
    rep_len = case.seq_lens.repeat_interleave(nq)
    want, want_lse = oracle.decode_paged(q.view(B * nq, hq, 128).float().numpy(), cache, rep_bt.numpy(),
                                         rep_len.numpy(), golden["signs_seed42_d128"], SCALE, return_lse=True)
    cache_d = torch.from_numpy(cache).to(DEV)
    rows, rows_lse = run_decode(q.view(B * nq, hq, 128).to(DEV), cache_d, rep_bt.to(DEV), rep_len.to(DEV),
                                want_lse=True)
    for ctas in (0, 3):
        ws = torch.zeros(_cabi.decode_workspace_bytes(B, nq * hq, hkv, 128, ctas), dtype=torch.uint8, device=DEV)
        out = torch.full((B, nq, hq, 128), float("nan"), dtype=torch.float16, device=DEV)
        lse = torch.empty(B, nq, hq, dtype=torch.float32, device=DEV)
        _cabi.decode_paged_multi(q.to(DEV), cache_d, case.block_table.to(DEV), case.seq_lens.to(DEV), signs_dev(),
                                 SCALE, ws, out, out_lse=lse, num_ctas=ctas)
        torch.cuda.synchronize()
        assert ws[:4].view(torch.int32).item() == 0
        got = out.float().cpu().numpy().reshape(B * nq, hq, 128)
        assert_attention_close(got, want, f"shared KV nq={nq} ctas={ctas}")
        assert_attention_close(got, rows.float().cpu().numpy(), f"shared KV vs repeated rows nq={nq}")
        assert (got.reshape(B, nq, hq, 128)[1] == 0).all()
        ok = np.isfinite(want_lse)
        np.testing.assert_allclose(lse.cpu().numpy().reshape(B * nq, hq)[ok], want_lse[ok], atol=2e-3)


@pytest.mark.parametrize("nq,hq,hkv", [(8, 32, 8), (5, 32, 8), (2, 8, 4), (1, 32, 8), (16, 4, 2), (4, 16, 16)])
def test_causal_queries_match_rows_of_their_own_length(oracle, golden, nq, hq, hkv):
    """tq_decode_paged_causal: the queries of a row are the last tokens of its sequence; query i must
    equal a plain decode row of length seq_len - (nq - 1 - i) (the oracle with one batch row per
    query).  Lengths around page, tile and query-count boundaries, one shorter than the queries."""
    lens = [40, 3, 1000, 16, 2100, 129, 128, 0]
    B = len(lens)
    case = synthetic.decode_case(seed=91 + nq, seq_lens=lens, heads=(hq, hkv), dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    g = torch.Generator().manual_seed(6)
    q = torch.randn(B, nq, hq, 128, generator=g).to(torch.float16)
    rep_bt = case.block_table.repeat_interleave(nq, dim=0)
    off = torch.arange(nq - 1, -1, -1, dtype=torch.int32).repeat(B)
    rep_len = (case.seq_lens.repeat_interleave(nq) - off).clamp(min=0)
    want, want_lse = oracle.decode_paged(q.view(B * nq, hq, 128).float().numpy(), cache, rep_bt.numpy(),
                                         rep_len.numpy(), golden["signs_seed42_d128"], SCALE, return_lse=True)
    cache_d = torch.from_numpy(cache).to(DEV)
    for ctas in (0, 5):
        ws = torch.zeros(_cabi.decode_workspace_bytes(B, nq * hq, hkv, 128, ctas), dtype=torch.uint8, device=DEV)
        out = torch.full((B, nq, hq, 128), float("nan"), dtype=torch.float16, device=DEV)
        lse = torch.empty(B, nq, hq, dtype=torch.float32, device=DEV)
        _cabi.decode_paged_causal(q.to(DEV), cache_d, case.block_table.to(DEV), case.seq_lens.to(DEV), signs_dev(),
                                  SCALE, ws, out, out_lse=lse, num_ctas=ctas)
        torch.cuda.synchronize()
        assert ws[:4].view(torch.int32).item() == 0
        got = out.float().cpu().numpy().reshape(B * nq, hq, 128)
        assert_attention_close(got, want, f"causal nq={nq} ctas={ctas}")
        empty = (rep_len == 0).numpy()
        assert (got[empty] == 0).all()
        ok = np.isfinite(want_lse)
        np.testing.assert_allclose(lse.cpu().numpy().reshape(B * nq, hq)[ok], want_lse[ok], atol=2e-3)
        assert np.isneginf(lse.cpu().numpy().reshape(B * nq, hq)[~ok]).all()


def test_causal_chunk_as_rows_sharing_a_page_table(oracle, golden):
    """A 40-token chunk after 1000 cached tokens as five rows of eight causal queries: the rows share
    the sequence's page table and differ in seq_lens."""
    total, chunk, nq = 1040, 40, 8
    case = synthetic.decode_case(seed=5, seq_lens=[total], heads=(32, 8), dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    g = torch.Generator().manual_seed(7)
    q = torch.randn(chunk, 32, 128, generator=g).to(torch.float16)
    lens_q = torch.arange(total - chunk + 1, total + 1, dtype=torch.int32)       # what each query token sees
    want = oracle.decode_paged(q.float().numpy(), cache, case.block_table.repeat(chunk, 1).numpy(), lens_q.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    rows = chunk // nq
    row_lens = lens_q[nq - 1::nq].contiguous()
    ws = torch.zeros(_cabi.decode_workspace_bytes(rows, nq * 32, 8), dtype=torch.uint8, device=DEV)
    out = torch.empty(rows, nq, 32, 128, dtype=torch.float16, device=DEV)
    _cabi.decode_paged_causal(q.view(rows, nq, 32, 128).to(DEV), torch.from_numpy(cache).to(DEV),
                              case.block_table.repeat(rows, 1).contiguous().to(DEV), row_lens.to(DEV), signs_dev(), SCALE, ws, out)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    assert_attention_close(out.float().cpu().numpy().reshape(chunk, 32, 128), want, "40-token chunk over 1000 cached tokens")


def test_wide_tile_csr_table_and_kv_windows(oracle, golden):
    """The wide-tile kernel (8 queries x GQA 4 = 32 columns) with a CSR page table, and as
    rotated partials over KV windows merged by tq_merge_rotated (the multi-GPU contract)."""
    lens = [1500, 90, 0, 300]
    B, nq, hq = len(lens), 8, 32
    case = synthetic.decode_case(seed=61, seq_lens=lens, dtype=torch.bfloat16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    q = torch.randn(B, nq, hq, 128, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    rep_bt = case.block_table.repeat_interleave(nq, dim=0)
    rep_len = case.seq_lens.repeat_interleave(nq)
    want, want_lse = oracle.decode_paged(q.view(B * nq, hq, 128).float().numpy(), cache, rep_bt.numpy(), rep_len.numpy(),
                                         golden["signs_seed42_d128"], SCALE, return_lse=True)
    cache_d, qd, sl = torch.from_numpy(cache).to(DEV), q.to(DEV), case.seq_lens.to(DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, nq * hq, 8), dtype=torch.uint8, device=DEV)
    # CSR table
    pages = [(int(n) + 15) // 16 for n in lens]
    indptr = torch.tensor([0] + list(np.cumsum(pages)), dtype=torch.int32, device=DEV)
    indices = torch.cat([case.block_table[b, :p] for b, p in enumerate(pages)]).to(torch.int32).to(DEV)
    out = torch.full((B, nq, hq, 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    _cabi.decode_paged_multi(qd, cache_d, indices, sl, signs_dev(), SCALE, ws, out, page_indptr=indptr)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    assert_attention_close(out.float().cpu().numpy().reshape(B * nq, hq, 128), want, "wide tile, CSR table")
    # KV windows -> rotated partials -> merge
    windows = [(0, 512), (512, 1024), (1024, -1), (2048, -1)]
    po = torch.empty(len(windows), B * nq, hq, 128, dtype=torch.float32, device=DEV)
    pl = torch.empty(len(windows), B * nq, hq, dtype=torch.float32, device=DEV)
    bt = case.block_table.to(DEV)
    for i, (a, b) in enumerate(windows):
        _cabi.decode_paged_multi(qd, cache_d, bt, sl, signs_dev(), SCALE, ws, po[i].view(B, nq, hq, 128),
                                 out_lse=pl[i].view(B, nq, hq), kv_begin=a, kv_end=b, rotated_partial=True)
    assert torch.isneginf(pl[3]).all()
    merged = torch.empty(B * nq, hq, 128, dtype=torch.float32, device=DEV)
    lse = torch.empty(B * nq, hq, dtype=torch.float32, device=DEV)
    _cabi.merge_rotated(po, pl, signs_dev(), merged, lse)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    assert_attention_close(merged.cpu().numpy(), want, "wide tile, merged windows")
    ok = np.isfinite(want_lse)
    np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=2e-3)


def test_wide_tile_many_short_sequences(oracle, golden):
    """120 short sequences (empty ones among them) with 8 shared-KV queries each: many segments per
    thread block in the wide-tile kernel, plain and causal."""
    rng = np.random.default_rng(11)
    lens = [int(x) for x in rng.integers(0, 150, size=120)]
    B, nq, hq = len(lens), 8, 32
    case = synthetic.decode_case(seed=34, seq_lens=lens, dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    q = torch.randn(B, nq, hq, 128, generator=torch.Generator().manual_seed(12)).to(torch.float16)
    rep_bt = case.block_table.repeat_interleave(nq, dim=0)
    cache_d, bt, sl = torch.from_numpy(cache).to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV)
    for causal in (False, True):
        off = torch.arange(nq - 1, -1, -1, dtype=torch.int32).repeat(B) if causal else torch.zeros(B * nq, dtype=torch.int32)
        rep_len = (case.seq_lens.repeat_interleave(nq) - off).clamp(min=0)
        want = oracle.decode_paged(q.view(B * nq, hq, 128).float().numpy(), cache, rep_bt.numpy(), rep_len.numpy(),
                                   golden["signs_seed42_d128"], SCALE)
        for ctas in (0, 8):
            ws = torch.zeros(_cabi.decode_workspace_bytes(B, nq * hq, 8, 128, ctas), dtype=torch.uint8, device=DEV)
            out = torch.full((B, nq, hq, 128), float("nan"), dtype=torch.float16, device=DEV)
            fn = _cabi.decode_paged_causal if causal else _cabi.decode_paged_multi
            fn(q.to(DEV), cache_d, bt, sl, signs_dev(), SCALE, ws, out, num_ctas=ctas)
            torch.cuda.synchronize()
            assert ws[:4].view(torch.int32).item() == 0
            assert_attention_close(out.float().cpu().numpy().reshape(B * nq, hq, 128), want,
                                   f"120 short sequences x 8 queries, causal={causal}, ctas={ctas}")


def test_shared_kv_rejects_more_than_32_columns():
    assert _cabi.decode_max_queries_per_seq(32, 8) == 8
    q = torch.zeros(1, 9, 32, 128, dtype=torch.float16, device=DEV)
    cache = torch.zeros(2, 4, 16, 8, 80, dtype=torch.uint8, device=DEV)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    sl = torch.ones(1, dtype=torch.int32, device=DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(1, 288, 8, 128, 0), dtype=torch.uint8, device=DEV)
    with pytest.raises(_cabi.TurboQuantError, match="queries_per_seq"):
        _cabi.decode_paged_multi(q, cache, bt, sl, signs_dev(), SCALE, ws, torch.empty_like(q))


def test_many_short_sequences(oracle, golden):
    """A large batch of short sequences (several sequences per thread block, empty ones among them)."""
    rng = np.random.default_rng(5)
    lens = [int(x) for x in rng.integers(0, 200, size=300)]
    case = synthetic.decode_case(seed=33, seq_lens=lens, dtype=torch.float16)
    cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    want = oracle.decode_paged(case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    for ctas in (0, 7):
        out = run_decode(case.q.to(DEV), torch.from_numpy(cache).to(DEV), case.block_table.to(DEV),
                         case.seq_lens.to(DEV), num_ctas=ctas)
        assert_attention_close(out.float().cpu().numpy(), want, f"300 short sequences, ctas={ctas}")


def test_too_many_sequences_per_block_is_reported():
    """More than 96 sequences inside one block's page range: status 2 in the workspace, no fault."""
    B = 200
    cache = torch.zeros(2, B, 16, 8, 80, dtype=torch.uint8, device=DEV)
    bt = torch.arange(B, dtype=torch.int32, device=DEV).view(B, 1)
    sl = torch.full((B,), 5, dtype=torch.int32, device=DEV)
    q = torch.zeros(B, 32, 128, dtype=torch.float16, device=DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, 32, 8, 128, 1), dtype=torch.uint8, device=DEV)
    out = torch.empty_like(q)
    _cabi.decode_paged(q, cache, bt, sl, signs_dev(), SCALE, ws, out, num_ctas=1)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 2
