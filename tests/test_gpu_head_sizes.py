"""Head sizes 64 and 256 (the reference's qwen3-0.6b and gemma-2 presets) and an odd size through
the paged write, decode, dequantization and page moves: bit-exact writes against the oracle and
the reference-generated quantizer fixtures, attention against the dequant-attention oracle."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape, slot_bytes
from tests.gpu_util import DEV, assert_attention_close

pytestmark = pytest.mark.gpu


def _signs(golden, d):
    pd = 1 << (d - 1).bit_length()
    key = f"signs_seed42_d{pd}"
    return torch.from_numpy(golden[key]) if key in golden.files else synthetic.make_signs(pd, 42)


@pytest.mark.parametrize("d", [64, 256])
def test_write_matches_reference_quantizer_fixture(golden, oracle, d):
    rows = torch.from_numpy(golden[f"q_rows_d{d}"])
    n = rows.shape[0] // 8 * 8
    k = rows[:n].reshape(n // 8, 8, d)
    sb = slot_bytes(d)
    assert sb == {64: 48, 256: 144}[d]
    nb = (n // 8 + 15) // 16
    cache = torch.zeros((2, nb, 16, 8, sb), dtype=torch.uint8, device=DEV)
    slots = torch.arange(n // 8, dtype=torch.int64)
    signs = _signs(golden, d)
    _cabi.write_kv_cache(cache, k.to(DEV), k.to(DEV), signs.to(DEV), slots.to(DEV), d)
    got = cache.cpu().numpy()[0].reshape(-1, sb)[:n]
    np.testing.assert_array_equal(got[:, :d // 2], oracle.low_first_to_cache_order(golden[f"q_packed_d{d}"][:n]))
    want_n = torch.from_numpy(golden[f"q_norms_d{d}"][:n]).to(torch.float16).numpy()
    for c in range(d // 64):
        np.testing.assert_array_equal(got[:, d // 2 + 2 * c:d // 2 + 2 * c + 2].copy().view(np.uint16).reshape(-1),
                                      want_n.view(np.uint16))
    assert (got[:, d // 2 + 2 * (d // 64):] == 0).all()              # pad untouched


@pytest.mark.parametrize("d,hq,hkv", [(64, 16, 8), (256, 16, 8), (256, 8, 4), (80, 8, 2), (192, 4, 4)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_write_decode_dequant_vs_oracle(oracle, golden, d, hq, hkv, dtype):
    lens = [1, 47, 0, 300, 1030]
    case = synthetic.decode_case(seed=200 + d + hq, seq_lens=lens, dtype=dtype, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    sb = slot_bytes(d)
    scale = 1.0 / math.sqrt(d)
    want_cache = np.zeros((2, case.num_blocks, 16, hkv, sb), np.uint8)
    oracle.write_kv_cache(want_cache, case.k.float().numpy(), case.v.float().numpy(), signs.numpy(),
                          case.slot_mapping.numpy(), d)
    attn = TurboQuantPagedAttention(hq, d, scale, hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    assert cache.shape[-1] == sb
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    np.testing.assert_array_equal(cache.cpu().numpy(), want_cache)
    want, want_lse = oracle.decode_paged(case.q.float().numpy(), want_cache, case.block_table.numpy(),
                                         case.seq_lens.numpy(), signs.numpy(), scale, return_lse=True)
    for ctas in (0, 3):
        attn_c = TurboQuantPagedAttention(hq, d, scale, hkv, num_ctas=ctas)
        out = torch.full(case.q.shape, float("nan"), dtype=torch.float32, device=DEV)
        lse = torch.empty(case.q.shape[:2], dtype=torch.float32, device=DEV)
        attn_c.decode(case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV), out, out_lse=lse)
        torch.cuda.synchronize()
        assert attn_c.status(len(lens), DEV) == 0
        got = out.cpu().numpy()
        assert_attention_close(got, want, f"head size {d}, {hq}/{hkv} heads, ctas={ctas}")
        assert (got[2] == 0).all()
        ok = np.isfinite(want_lse)
        np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=2e-3)
    # bulk dequantization of the cached tokens: bit-identical to the oracle in fp32
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    k_out, v_out = attn.dequant_cached(cache, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, sum(lens), dtype=torch.float32)
    torch.cuda.synchronize()
    at = 0
    for b, n in enumerate(lens):
        t = np.arange(n)
        pages = case.block_table.numpy()[b, t // 16]
        for which, got_t in ((0, k_out), (1, v_out)):
            want_rows = oracle.dequant_cache_rows(want_cache[which, pages, t % 16], signs.numpy(), d)
            np.testing.assert_array_equal(got_t[at:at + n].cpu().numpy(), want_rows)
        at += n


@pytest.mark.parametrize("d", [64, 256])
def test_page_offload_round_trip(d):
    hkv = 4
    attn = TurboQuantPagedAttention(8, d, 1.0 / math.sqrt(d), hkv)
    g = torch.Generator().manual_seed(d)
    cache = torch.randint(0, 256, kv_cache_shape(12, 16, hkv, d), dtype=torch.uint8, generator=g).to(DEV)
    ids = torch.tensor([7, 2, 11], dtype=torch.int32, device=DEV)
    host = attn.offload_pages(cache, ids)
    torch.cuda.synchronize()
    other = torch.zeros_like(cache)
    dst = torch.tensor([0, 5, 1], dtype=torch.int32, device=DEV)
    attn.restore_pages(other, dst, host)
    torch.cuda.synchronize()
    payload = d // 2 + 2 * (d // 64)
    a, b = cache.cpu().numpy(), other.cpu().numpy()
    for s, t in zip((7, 2, 11), (0, 5, 1)):
        np.testing.assert_array_equal(b[:, t, ..., :payload], a[:, s, ..., :payload])
    assert (b[:, [2, 3, 4, 6]] == 0).all()


def test_rejected_geometries():
    with pytest.raises(_cabi.TurboQuantError, match="head_size"):
        TurboQuantPagedAttention(8, 16, 0.25, 8)
    attn = TurboQuantPagedAttention(32, 64, 0.125, 2)               # 16 query heads per KV head
    cache = torch.zeros(kv_cache_shape(2, 16, 2, 64), dtype=torch.uint8, device=DEV)
    q = torch.zeros(1, 32, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(_cabi.TurboQuantError, match="query heads per KV head"):
        attn.decode(q, cache, torch.zeros(1, 2, dtype=torch.int32, device=DEV), torch.ones(1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("d,sb", [(64, 52), (256, 150)])
def test_slots_that_are_not_16_byte_multiples_take_the_plain_kernel(oracle, golden, d, sb):
    """The tensor-core decode kernel for these head sizes reads codes with 16-byte loads; a cache
    whose slots are not a multiple of 16 bytes (a caller's own padding) falls back to the plain
    kernel and must give the same answer."""
    lens, hq, hkv = [33, 700], 8, 4
    case = synthetic.decode_case(seed=300 + d, seq_lens=lens, dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    scale = 1.0 / math.sqrt(d)
    cache_np = np.zeros((2, case.num_blocks, 16, hkv, sb), np.uint8)
    oracle.write_kv_cache(cache_np, case.k.float().numpy(), case.v.float().numpy(), signs.numpy(), case.slot_mapping.numpy(), d)
    want = oracle.decode_paged(case.q.float().numpy(), cache_np, case.block_table.numpy(), case.seq_lens.numpy(), signs.numpy(), scale)
    cache = torch.zeros((2, case.num_blocks, 16, hkv, sb), dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, case.k.to(DEV), case.v.to(DEV), signs.to(DEV), case.slot_mapping.to(DEV), d)
    np.testing.assert_array_equal(cache.cpu().numpy(), cache_np)
    ws = torch.zeros(_cabi.decode_workspace_bytes(len(lens), hq, hkv, d, 0), dtype=torch.uint8, device=DEV)
    out = torch.empty(case.q.shape, dtype=torch.float32, device=DEV)
    _cabi.decode_paged(case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV), signs.to(DEV), scale, ws, out)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    assert_attention_close(out.cpu().numpy(), want, f"head size {d}, slots of {sb} bytes")
    # bulk dequantization out of the odd-sized slots: byte loads instead of vector loads, same values
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device=DEV)
    k_out = torch.empty(sum(lens), hkv, d, dtype=torch.float32, device=DEV)
    v_out = torch.empty_like(k_out)
    _cabi.dequant_paged(cache, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, signs.to(DEV), k_out, v_out,
                        max_pages=case.block_table.shape[-1])
    torch.cuda.synchronize()
    at = 0
    for b, n in enumerate(lens):
        t = np.arange(n)
        pages = case.block_table.numpy()[b, t // 16]
        for which, got_t in ((0, k_out), (1, v_out)):
            want_rows = oracle.dequant_cache_rows(cache_np[which, pages, t % 16][..., :slot_bytes(d)], signs.numpy(), d)
            np.testing.assert_array_equal(got_t[at:at + n].cpu().numpy(), want_rows)
        at += n


@pytest.mark.parametrize("d,hkv", [(64, 8), (256, 4), (80, 2), (72, 3), (192, 4)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dequant_16_bit_outputs_are_the_rounded_fp32_ones(golden, d, hkv, dtype):
    """The 16-bit outputs leave as packed 16-byte stores where the rows allow it (head size 72: they do not);
    every element must be the fp32 result rounded once."""
    lens = [5, 0, 130, 64]
    case = synthetic.decode_case(seed=400 + d, seq_lens=lens, dtype=torch.float16, heads=(hkv, hkv), head_dim=d)
    attn = TurboQuantPagedAttention(hkv, d, 1.0 / math.sqrt(d), hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    args = (cache, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, sum(lens))
    k32, v32 = attn.dequant_cached(*args, dtype=torch.float32)
    k16, v16 = attn.dequant_cached(*args, dtype=dtype)
    torch.cuda.synchronize()
    assert torch.equal(k16, k32.to(dtype)) and torch.equal(v16, v32.to(dtype))
    assert k32.abs().max().item() > 0


@pytest.mark.parametrize("d,hq,hkv", [(64, 16, 8), (256, 8, 4)])
def test_kv_windows_partials_and_merge(oracle, golden, d, hq, hkv):
    """The KV-axis split contract for these head sizes: rotated partials over token windows, merged by
    tq_merge_rotated, equal the one-call decode and the oracle; with a CSR page table."""
    lens = [1500, 90]
    case = synthetic.decode_case(seed=500 + d, seq_lens=lens, dtype=torch.bfloat16, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    scale = 1.0 / math.sqrt(d)
    attn = TurboQuantPagedAttention(hq, d, scale, hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    q, sl = case.q.to(DEV), case.seq_lens.to(DEV)
    pages = [(n + 15) // 16 for n in lens]
    indptr = torch.tensor([0, pages[0], pages[0] + pages[1]], dtype=torch.int32, device=DEV)
    indices = torch.cat([case.block_table[b, :p] for b, p in enumerate(pages)]).to(torch.int32).to(DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(2, hq, hkv, d, 0), dtype=torch.uint8, device=DEV)
    full = torch.empty(2, hq, d, dtype=torch.float32, device=DEV)
    _cabi.decode_paged(q, cache, indices, sl, signs.to(DEV), scale, ws, full, page_indptr=indptr)
    windows = [(0, 512), (512, 1024), (1024, -1), (2048, -1)]          # the last one is empty
    po = torch.empty(len(windows), 2, hq, d, dtype=torch.float32, device=DEV)   # d is the padded width here
    pl = torch.empty(len(windows), 2, hq, dtype=torch.float32, device=DEV)
    for i, (a, b) in enumerate(windows):
        _cabi.decode_paged_partial(q, cache, indices, sl, signs.to(DEV), scale, ws, po[i], pl[i], kv_begin=a, kv_end=b,
                                   page_indptr=indptr)
    assert torch.isneginf(pl[3]).all() and torch.isneginf(pl[1, 1]).all()
    out = torch.empty(2, hq, d, dtype=torch.float32, device=DEV)
    lse = torch.empty(2, hq, dtype=torch.float32, device=DEV)
    _cabi.merge_rotated(po, pl, signs.to(DEV), out, lse)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    np.testing.assert_allclose(out.cpu().numpy(), full.cpu().numpy(), atol=3e-4, rtol=1e-3)
    want_cache = cache.cpu().numpy()
    want, want_lse = oracle.decode_paged(case.q.float().numpy(), want_cache, case.block_table.numpy(), case.seq_lens.numpy(),
                                         signs.numpy(), scale, return_lse=True)
    assert_attention_close(out.cpu().numpy(), want, f"head size {d}: merged windows")
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=2e-3)


@pytest.mark.parametrize("d,hq,hkv", [(96, 32, 8), (64, 16, 8), (80, 8, 2)])
def test_kv_split_helper_sizes_partials_by_the_padded_head(monkeypatch, d, hq, hkv):
    """parallel.kv_split_decode with a one-rank group (the collective replaced by a copy): the rotated partial
    it allocates must be as wide as the padded head, and partial + merge must equal the plain decode."""
    import torch.distributed as dist
    from turboquant_b200 import parallel
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 1)
    monkeypatch.setattr(dist, "all_gather_into_tensor", lambda out, inp, group=None: out.copy_(inp))
    lens = [700, 33]
    case = synthetic.decode_case(seed=600 + d, seq_lens=lens, dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    attn = TurboQuantPagedAttention(hq, d, 1.0 / math.sqrt(d), hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    q, bt, sl = case.q.to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV)
    want = torch.empty(len(lens), hq, d, dtype=torch.float32, device=DEV)
    attn.decode(q, cache, bt, sl, want)
    guard = torch.full((3, len(lens), hq, d), 7.0, dtype=torch.float32, device=DEV)   # neighbours of the output
    parallel.kv_split_decode(attn, q, cache, bt, sl, guard[1])
    torch.cuda.synchronize()
    assert (guard[0] == 7.0).all() and (guard[2] == 7.0).all()
    np.testing.assert_allclose(guard[1].cpu().numpy(), want.cpu().numpy(), atol=3e-4, rtol=1e-3)


@pytest.mark.parametrize("d,hkv", [(64, 2), (256, 1), (80, 3)])
def test_dequant_of_a_large_job(oracle, golden, d, hkv):
    """From 16384 token positions on, a lane group of the dequantizer walks all rows of its token instead of
    taking one row: same values, bit for bit, including the second sequence's ragged end."""
    lens = [9000, 7001]
    case = synthetic.decode_case(seed=700 + d, seq_lens=lens, dtype=torch.float16, heads=(hkv, hkv), head_dim=d)
    assert len(lens) * case.block_table.shape[1] * 16 >= 16384
    signs = _signs(golden, d)
    attn = TurboQuantPagedAttention(hkv, d, 1.0 / math.sqrt(d), hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    k_out, v_out = attn.dequant_cached(cache, case.block_table.to(DEV), case.seq_lens.to(DEV), cu, sum(lens), dtype=torch.float32)
    torch.cuda.synchronize()
    cache_np = cache.cpu().numpy()
    at = 0
    for b, n in enumerate(lens):
        t = np.arange(n)
        pages = case.block_table.numpy()[b, t // 16]
        for which, got_t in ((0, k_out), (1, v_out)):
            want_rows = oracle.dequant_cache_rows(cache_np[which, pages, t % 16], signs.numpy(), d)
            np.testing.assert_array_equal(got_t[at:at + n].cpu().numpy(), want_rows)
        at += n


@pytest.mark.parametrize("d,hkv", [(64, 3), (256, 2), (80, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_write_edge_cases(oracle, golden, monkeypatch, d, hkv, dtype):
    """The write of these head sizes on what an engine hands it: K / V as strided views of one fused tensor,
    int32 and int64 slot ids, skipped (-1) and out-of-range slots (dropped and counted), a token count that is not
    a multiple of the four rows a warp takes, degenerate rows; pad bytes untouched unless asked for."""
    monkeypatch.delenv("TQ_DEBUG_CHECKS", raising=False)   # the device-side handling is what is tested
    T, nb = 203, 16
    g = torch.Generator().manual_seed(800 + d)
    fused = torch.randn(T, 3 * hkv * d, generator=g).to(dtype)
    fused[5, hkv * d:hkv * d + d] = 0                      # an all-zero K row: norm clamp
    fused[6, hkv * d:hkv * d + d] = 1e-30                  # tiny values: the division instruction's path
    fused[7, hkv * d + 3] = float("inf")                   # a non-finite row
    fused[8, hkv * d:hkv * d + d] = 3.0                    # a constant row
    key = fused[:, hkv * d:2 * hkv * d].view(T, hkv, d)
    value = fused[:, 2 * hkv * d:].view(T, hkv, d)
    assert key.stride(0) == 3 * hkv * d
    slots = torch.randperm(nb * 16, generator=g)[:T]
    slots[10] = -1
    slots[50] = -1
    bad = slots.clone()
    bad[20] = nb * 16
    bad[120] = 2 ** 40
    sb = slot_bytes(d)
    signs = _signs(golden, d)
    ok = bad.clone()
    ok[[20, 120]] = -1
    for zero_pad in (False, True):
        want = np.full((2, nb, 16, hkv, sb), 0xEE, np.uint8)
        oracle.write_kv_cache(want, key.float().numpy(), value.float().numpy(), signs.numpy(), ok.numpy(), d)
        before = _cabi.fault_counts()[0]
        cache = torch.full((2, nb, 16, hkv, sb), 0xEE, dtype=torch.uint8, device=DEV)
        fused_dev = fused.to(DEV)
        _cabi.write_kv_cache(cache, fused_dev[:, hkv * d:2 * hkv * d].view(T, hkv, d), fused_dev[:, 2 * hkv * d:].view(T, hkv, d),
                             signs.to(DEV), bad.to(DEV), d, zero_pad=zero_pad)
        torch.cuda.synchronize()
        assert _cabi.fault_counts()[0] - before == 2
        got = cache.cpu().numpy()
        pd = 1 << (d - 1).bit_length() if d > 64 else 64
        used = pd // 2 + 2 * (pd // 64)
        np.testing.assert_array_equal(got[..., :used], want[..., :used])
        written = np.zeros((nb * 16,), bool)
        written[ok[ok >= 0].numpy()] = True
        pad = got.reshape(2, nb * 16, hkv, sb)[..., used:]
        if used < sb:
            assert (pad[:, ~written] == 0xEE).all()
            assert (pad[:, written] == (0 if zero_pad else 0xEE)).all()
    # int32 slot ids take the same path
    cache32 = torch.full((2, nb, 16, hkv, sb), 0xEE, dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache32, fused_dev[:, hkv * d:2 * hkv * d].view(T, hkv, d), fused_dev[:, 2 * hkv * d:].view(T, hkv, d),
                         signs.to(DEV), ok.to(torch.int32).to(DEV), d, zero_pad=True)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(cache32.cpu().numpy(), got)


@pytest.mark.parametrize("d", [64, 256])
def test_page_ids_and_lengths_that_cannot_be_trusted(oracle, golden, monkeypatch, d):
    """Index validation of the kernels for these head sizes: a page id outside the cache is status 5 in the
    decode (the access is skipped, other sequences are unaffected) and a counted skip in the dequantizer; a
    sequence longer than its page table is status 4 and reads nothing."""
    monkeypatch.delenv("TQ_DEBUG_CHECKS", raising=False)   # the device-side handling is what is tested
    hq, hkv = 8, 4
    case = synthetic.decode_case(seed=900 + d, seq_lens=[200, 900, 48], dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    scale = 1.0 / math.sqrt(d)
    attn = TurboQuantPagedAttention(hq, d, scale, hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    cache_np = cache.cpu().numpy()
    want = oracle.decode_paged(case.q.float().numpy(), cache_np, case.block_table.numpy(), case.seq_lens.numpy(), signs.numpy(), scale)
    q, sl = case.q.to(DEV), case.seq_lens.to(DEV)

    def run(bt, lens):
        ws = torch.zeros(_cabi.decode_workspace_bytes(3, hq, hkv, d, 0), dtype=torch.uint8, device=DEV)
        out = torch.zeros(3, hq, d, dtype=torch.float32, device=DEV)
        _cabi.decode_paged(q, cache, bt, lens, signs.to(DEV), scale, ws, out)
        torch.cuda.synchronize()
        return out.cpu().numpy(), int(ws[:4].view(torch.int32).item())

    good, status = run(case.block_table.to(DEV), sl)
    assert status == 0
    assert_attention_close(good, want, f"head size {d}, in-range page table")
    for bad_id in (case.num_blocks, -1, 2 ** 31 - 1):
        bt = case.block_table.clone()
        bt[1, 3] = bad_id
        out, status = run(bt.to(DEV), sl)
        assert status == 5, (bad_id, status)
        assert np.isfinite(out).all()
        assert_attention_close(out[[0, 2]], want[[0, 2]], f"head size {d}, rows beside the bad page id {bad_id}")
    too_long = torch.tensor([200, 900, 48 + 16 * case.block_table.shape[1]], dtype=torch.int32, device=DEV)
    out, status = run(case.block_table.to(DEV), too_long)
    assert status == 4 and (out[2] == 0).all()
    assert_attention_close(out[:2], want[:2], f"head size {d}, rows beside the over-long one")
    # dequantization: the bad page's rows stay unwritten and are counted once
    bt = case.block_table.clone()
    bt[0, 2] = case.num_blocks + 3
    lens = [200, 900, 48]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    k = torch.full((sum(lens), hkv, d), 7.0, dtype=torch.float32, device=DEV)
    v = torch.full_like(k, 7.0)
    before = _cabi.fault_counts()
    _cabi.dequant_paged(cache, bt.to(DEV), sl, cu, signs.to(DEV), k, v)
    torch.cuda.synchronize()
    assert _cabi.fault_counts()[1] - before[1] == 1
    kk = k.cpu().numpy()
    assert (kk[32:48] == 7.0).all()
    t = np.arange(32)
    want_rows = oracle.dequant_cache_rows(cache_np[0, case.block_table.numpy()[0, t // 16], t % 16], signs.numpy(), d)
    assert np.array_equal(kk[:32], want_rows)


@pytest.mark.parametrize("d,hq,hkv,nq", [(64, 8, 4, 4), (64, 16, 8, 2), (256, 4, 4, 7), (80, 4, 2, 3)])
def test_queries_that_share_a_sequence(oracle, golden, d, hq, hkv, nq):
    """Several decode queries per sequence (speculative tokens verified without a causal mask, or any caller that
    would repeat the sequence as batch rows) ride as extra columns of the KV heads: up to 8 columns per KV head at
    these head sizes.  Against the oracle with the rows repeated; rotated partials over windows merge to the same."""
    lens = [700, 0, 33]
    B = len(lens)
    case = synthetic.decode_case(seed=1000 + d + nq, seq_lens=lens, dtype=torch.bfloat16, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    scale = 1.0 / math.sqrt(d)
    attn = TurboQuantPagedAttention(hq, d, scale, hkv)
    assert _cabi.decode_max_queries_per_seq(hq, hkv, d) >= nq
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    q = torch.randn(B, nq, hq, d, generator=torch.Generator().manual_seed(nq)).to(torch.bfloat16)
    bt, sl = case.block_table.to(DEV), case.seq_lens.to(DEV)
    lse = torch.empty(B, nq, hq, dtype=torch.float32, device=DEV)
    out = attn.decode_shared(q.to(DEV), cache, bt, sl, out_lse=lse)
    torch.cuda.synchronize()
    assert attn.status(B, DEV, nq) == 0
    rep_bt = np.repeat(case.block_table.numpy(), nq, axis=0)
    rep_sl = np.repeat(case.seq_lens.numpy(), nq)
    want, want_lse = oracle.decode_paged(q.float().numpy().reshape(B * nq, hq, d), cache.cpu().numpy(), rep_bt, rep_sl,
                                         signs.numpy(), scale, return_lse=True)
    assert_attention_close(out.float().cpu().numpy().reshape(B * nq, hq, d), want, f"head size {d}, {nq} queries per sequence")
    ok = np.isfinite(want_lse)
    np.testing.assert_allclose(lse.cpu().numpy().reshape(B * nq, hq)[ok], want_lse[ok], atol=2e-3)
    assert (out[1] == 0).all()
    # the same through rotated partials over two windows and the merge
    pd = 64 if d <= 64 else 128 if d <= 128 else 256
    ws = attn.workspace(B, DEV, nq)
    po = torch.empty(2, B, nq, hq, pd, dtype=torch.float32, device=DEV)
    pl = torch.empty(2, B, nq, hq, dtype=torch.float32, device=DEV)
    for i, (a, b) in enumerate([(0, 256), (256, -1)]):
        _cabi.decode_paged_multi(q.to(DEV), cache, bt, sl, signs.to(DEV), scale, ws, po[i], out_lse=pl[i],
                                 kv_begin=a, kv_end=b, rotated_partial=True)
    merged = torch.empty(B, nq, hq, d, dtype=torch.float32, device=DEV)
    _cabi.merge_rotated(po, pl, signs.to(DEV), merged)
    torch.cuda.synchronize()
    np.testing.assert_allclose(merged.cpu().numpy(), out.float().cpu().numpy(), atol=2e-3, rtol=1e-2)
    with pytest.raises(_cabi.TurboQuantError, match="queries_per_seq"):
        attn.decode_shared(torch.zeros(B, 8 // (hq // hkv) + 1, hq, d, dtype=torch.bfloat16, device=DEV), cache, bt, sl)


def test_shared_queries_through_the_plain_kernel(oracle, golden):
    """Slots that are not 16-byte multiples take the plain decode kernel; queries that share a sequence work there too."""
    d, sb, hq, hkv, nq, lens = 64, 52, 8, 4, 3, [33, 700]
    B = len(lens)
    case = synthetic.decode_case(seed=1100, seq_lens=lens, dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    signs = _signs(golden, d)
    scale = 1.0 / math.sqrt(d)
    cache_np = np.zeros((2, case.num_blocks, 16, hkv, sb), np.uint8)
    oracle.write_kv_cache(cache_np, case.k.float().numpy(), case.v.float().numpy(), signs.numpy(), case.slot_mapping.numpy(), d)
    q = torch.randn(B, nq, hq, d, generator=torch.Generator().manual_seed(5)).to(torch.float16)
    want = oracle.decode_paged(q.float().numpy().reshape(B * nq, hq, d), cache_np, np.repeat(case.block_table.numpy(), nq, axis=0),
                               np.repeat(case.seq_lens.numpy(), nq), signs.numpy(), scale)
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, nq * hq, hkv, d, 0), dtype=torch.uint8, device=DEV)
    out = torch.empty(B, nq, hq, d, dtype=torch.float32, device=DEV)
    _cabi.decode_paged_multi(q.to(DEV), torch.from_numpy(cache_np).to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV),
                             signs.to(DEV), scale, ws, out)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    assert_attention_close(out.cpu().numpy().reshape(B * nq, hq, d), want, "plain kernel, 3 queries per sequence")


@pytest.mark.parametrize("d,hkv", [(64, 2), (256, 1)])
def test_write_of_a_large_job(oracle, golden, d, hkv):
    """From 8192 tokens on, a lane group of the write kernel walks all rows of its token instead of taking one
    row: same bytes, with skipped tokens among them."""
    T, nb = 8200, 520
    g = torch.Generator().manual_seed(1200 + d)
    k = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    slots = torch.randperm(nb * 16, generator=g)[:T]
    slots[torch.randperm(T, generator=g)[:40]] = -1
    slots[100:104] = -1                                   # four neighbouring tokens: a whole warp pass is skipped
    signs = _signs(golden, d)
    want = np.zeros((2, nb, 16, hkv, slot_bytes(d)), np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), signs.numpy(), slots.numpy(), d)
    cache = torch.zeros(kv_cache_shape(nb, 16, hkv, d), dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, k.to(DEV), v.to(DEV), signs.to(DEV), slots.to(DEV), d)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(cache.cpu().numpy(), want)
