"""Index validation that cannot fault: stale or garbage slot ids, page ids and lengths are caught
by the kernels (dropped / skipped / replaced, with a sticky status or a counter) instead of being
turned into addresses, the host-side TQ_DEBUG_CHECKS mode raises before the launch, and a wait
for a peer that never pushes runs out within its (shortened) limit and reports status 1.

Every case also checks parity on the in-range part of the data: validation must not disturb it."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic
from tests.gpu_util import DEV, assert_attention_close, oracle_cache, signs_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128)


def test_write_drops_slots_beyond_the_cache(oracle, golden, monkeypatch):
    monkeypatch.delenv("TQ_DEBUG_CHECKS", raising=False)   # the device-side handling is what is tested
    k, v, slots, nb = synthetic.write_case(seed=12, num_tokens=300, num_skipped=5)
    bad = slots.clone()
    bad[7] = nb * 16                 # first slot past the end
    bad[100] = nb * 16 + 12345
    bad[250] = 2 ** 40               # garbage
    before = _cabi.fault_counts()[0]
    cache = torch.full((2, nb, 16, 8, 80), 0xEE, dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, k.to(DEV), v.to(DEV), signs_dev(), bad.to(DEV), 128)
    torch.cuda.synchronize()
    assert _cabi.fault_counts()[0] - before == 3
    want = np.full((2, nb, 16, 8, 80), 0xEE, np.uint8)
    ok = slots.clone()
    ok[[7, 100, 250]] = -1           # the oracle skips what the kernel must have dropped
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), golden["signs_seed42_d128"], ok.numpy(), 128)
    assert np.array_equal(cache.cpu().numpy(), want)
    # int32 slots take the same path
    cache2 = torch.full((2, nb, 16, 8, 80), 0xEE, dtype=torch.uint8, device=DEV)
    bad32 = bad.clamp(max=2 ** 31 - 1).to(torch.int32)
    _cabi.write_kv_cache(cache2, k.to(DEV), v.to(DEV), signs_dev(), bad32.to(DEV), 128)
    torch.cuda.synchronize()
    assert np.array_equal(cache2.cpu().numpy(), want)


def _decode(q, cache, bt, sl, **kw):
    B, Hq, _ = q.shape
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, Hq, cache.shape[3]), dtype=torch.uint8, device=DEV)
    out = torch.full((B, Hq, 128), float("nan"), dtype=torch.float32, device=DEV)
    _cabi.decode_paged(q, cache, bt, sl, signs_dev(), SCALE, ws, out, **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy(), int(ws[:4].view(torch.int32).item())


def test_decode_reports_page_ids_outside_the_cache(oracle, golden, monkeypatch):
    monkeypatch.delenv("TQ_DEBUG_CHECKS", raising=False)   # the device-side handling is what is tested
    case = synthetic.decode_case(seed=14, seq_lens=[200, 900, 48], dtype=torch.float16)
    cache_np = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    cache = torch.from_numpy(cache_np).to(DEV)
    q, sl = case.q.to(DEV), case.seq_lens.to(DEV)
    want = oracle.decode_paged(case.q.float().numpy(), cache_np, case.block_table.numpy(), case.seq_lens.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    good, status = _decode(q, cache, case.block_table.to(DEV), sl)
    assert status == 0
    assert_attention_close(good, want, "in-range page table")
    for bad_id in (case.num_blocks, -1, 2 ** 31 - 1):
        bt = case.block_table.clone()
        bt[1, 3] = bad_id
        out, status = _decode(q, cache, bt.to(DEV), sl)
        assert status == 5, (bad_id, status)
        assert np.isfinite(out).all()
        # the sequences that the bad id does not belong to are unaffected
        assert_attention_close(out[[0, 2]], want[[0, 2]], f"rows beside the bad page id {bad_id}")


def test_decode_reports_a_sequence_longer_than_its_page_table(oracle, golden, monkeypatch):
    monkeypatch.delenv("TQ_DEBUG_CHECKS", raising=False)   # the device-side handling is what is tested
    case = synthetic.decode_case(seed=15, seq_lens=[100, 64], dtype=torch.float16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    sl = torch.tensor([100, 64 + 16 * case.block_table.shape[1]], dtype=torch.int32, device=DEV)
    out, status = _decode(case.q.to(DEV), cache, case.block_table.to(DEV), sl)
    assert status == 4 and (out == 0).all()
    # the same through a CSR page list whose second span is too short
    pages = [7, 4]
    indptr = torch.tensor([0, 7, 11], dtype=torch.int32, device=DEV)
    indices = torch.cat([case.block_table[b, :p] for b, p in enumerate(pages)]).to(torch.int32).to(DEV)
    sl2 = torch.tensor([100, 65], dtype=torch.int32, device=DEV)      # 65 tokens need 5 pages, 4 are listed
    out, status = _decode(case.q.to(DEV), cache, indices, sl2, page_indptr=indptr, max_pages=1)
    assert status == 4 and (out == 0).all()


def test_dequant_and_page_moves_skip_ids_outside_the_cache(oracle, golden):
    case = synthetic.decode_case(seed=16, seq_lens=[40, 70], dtype=torch.float16)
    cache_np = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    cache = torch.from_numpy(cache_np).to(DEV)
    bt = case.block_table.clone()
    bt[1, 2] = case.num_blocks + 3
    cu = torch.tensor([0, 40, 110], dtype=torch.int32, device=DEV)
    k = torch.full((110, 8, 128), 7.0, dtype=torch.float32, device=DEV)
    v = torch.full_like(k, 7.0)
    before = _cabi.fault_counts()
    _cabi.dequant_paged(cache, bt.to(DEV), case.seq_lens.to(DEV), cu, signs_dev(), k, v)
    torch.cuda.synchronize()
    after = _cabi.fault_counts()
    assert after[1] - before[1] == 1
    kk = k.cpu().numpy()
    assert (kk[40 + 32:40 + 48] == 7.0).all()                 # the skipped page's rows stay unwritten
    t = np.arange(40)
    want = oracle.dequant_cache_rows(cache_np[0, case.block_table.numpy()[0, t // 16], t % 16],
                                     golden["signs_seed42_d128"], 128)
    assert np.array_equal(kk[:40], want)                      # the rest is bit-exact as ever
    ids = torch.tensor([0, case.num_blocks, 1, -5], dtype=torch.int32, device=DEV)
    packed = torch.full((_cabi.pages_packed_bytes(4, 16, 8),), 0xAB, dtype=torch.uint8, device=DEV)
    _cabi.pages_gather(cache, ids, packed)
    torch.cuda.synchronize()
    assert _cabi.fault_counts()[2] - before[2] == 2
    per = packed.numel() // 4
    pk = packed.cpu().numpy().reshape(4, per)
    assert (pk[1] == 0xAB).all() and (pk[3] == 0xAB).all() and not (pk[0] == 0xAB).all()


def test_host_side_debug_checks(monkeypatch):
    monkeypatch.setenv("TQ_DEBUG_CHECKS", "1")
    case = synthetic.decode_case(seed=17, seq_lens=[33], dtype=torch.float16)
    cache = torch.zeros((2, case.num_blocks, 16, 8, 80), dtype=torch.uint8, device=DEV)
    slots = case.slot_mapping.clone()
    slots[3] = case.num_blocks * 16
    with pytest.raises(_cabi.TurboQuantError, match="slot"):
        _cabi.write_kv_cache(cache, case.k.to(DEV), case.v.to(DEV), signs_dev(), slots.to(DEV), 128)
    ws = torch.zeros(_cabi.decode_workspace_bytes(1, 32, 8), dtype=torch.uint8, device=DEV)
    out = torch.empty(1, 32, 128, dtype=torch.float16, device=DEV)
    bt = case.block_table.clone()
    bt[0, 1] = -2
    with pytest.raises(_cabi.TurboQuantError, match="page id"):
        _cabi.decode_paged(case.q.to(DEV), cache, bt.to(DEV), case.seq_lens.to(DEV), signs_dev(), SCALE, ws, out)
    with pytest.raises(_cabi.TurboQuantError, match="pages"):
        _cabi.decode_paged(case.q.to(DEV), cache, case.block_table.to(DEV),
                           torch.tensor([4000], dtype=torch.int32, device=DEV), signs_dev(), SCALE, ws, out)
    _cabi.decode_paged(case.q.to(DEV), cache, case.block_table.to(DEV), case.seq_lens.to(DEV), signs_dev(), SCALE, ws, out)
    torch.cuda.synchronize()


def test_exchange_wait_for_a_silent_peer_runs_out(oracle, golden):
    """world = 2 on one GPU with a second buffer that no kernel ever pushes into as rank 1: the
    merge of rank 0 finds its own flag, waits for rank 1's within the shortened limit, gives up
    with status 1 and leaves `out` untouched.  Nothing waits on a kernel of the same GPU."""
    case = synthetic.decode_case(seed=18, seq_lens=[500], dtype=torch.float16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    q = case.q.to(DEV).view(1, 1, 32, 128)
    nbytes = _cabi.exchange_bytes(32, 2)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    silent = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    ws = torch.zeros(_cabi.decode_workspace_bytes(1, 32, 8), dtype=torch.uint8, device=DEV)
    out = torch.full((1, 1, 32, 128), 123.0, dtype=torch.float32, device=DEV)
    _cabi.set_exchange_wait_limit(2000)                       # x 256 ns: about half a millisecond
    try:
        _cabi.decode_paged_exchange(q, cache, case.block_table.to(DEV), case.seq_lens.to(DEV), signs_dev(), SCALE,
                                    ws, 0, [mine.data_ptr(), silent.data_ptr()], nbytes, out)
        torch.cuda.synchronize()
    finally:
        _cabi.set_exchange_wait_limit(0)
    assert int(mine[4:8].view(torch.int32).item()) == 1       # sticky status: a wait ran out
    assert (out == 123.0).all()
    assert int(ws[:4].view(torch.int32).item()) == 0          # the decode itself was fine
    flags_silent = silent[64:72].view(torch.int32).cpu().numpy()
    assert flags_silent[0] == 1 and flags_silent[1] == 0      # rank 0 did push into the peer's buffer


def test_rotated_partial_buffers_must_have_the_padded_width():
    """A rotated partial is as wide as the padded head (96 -> 128): a head_size-wide buffer would be written
    past its end, so the binding refuses it before the launch."""
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    d, hq, hkv = 96, 8, 2
    attn = TurboQuantPagedAttention(hq, d, 1.0 / math.sqrt(d), hkv)
    cache = torch.zeros(kv_cache_shape(4, 16, hkv, d), dtype=torch.uint8, device=DEV)
    q = torch.zeros(1, hq, d, dtype=torch.float16, device=DEV)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    sl = torch.full((1,), 20, dtype=torch.int32, device=DEV)
    ws = attn.workspace(1, DEV)
    lse = torch.empty(1, hq, dtype=torch.float32, device=DEV)
    with pytest.raises(_cabi.TurboQuantError, match="padded head size"):
        _cabi.decode_paged_partial(q, cache, bt, sl, attn.signs(DEV), attn.scale, ws,
                                   torch.empty(1, hq, d, dtype=torch.float32, device=DEV), lse)
    _cabi.decode_paged_partial(q, cache, bt, sl, attn.signs(DEV), attn.scale, ws,
                               torch.empty(1, hq, 128, dtype=torch.float32, device=DEV), lse)
    torch.cuda.synchronize()
