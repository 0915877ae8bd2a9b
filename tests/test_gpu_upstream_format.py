"""GPU parity of the upstream-format kernels (tq_nc_*) against the oracle's restatement."""
import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi
from oracle import tq_oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0") if torch.cuda.is_available() else None


def _case(seed, lens, H, Hq, d, dtype):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    k = torch.randn(total, H, d, generator=g).to(dtype)
    v = (torch.randn(total, H, d, generator=g) * 2 + 0.5).to(dtype)
    pages = [(n + 15) // 16 for n in lens]
    nb = sum(pages) + 3
    perm = torch.randperm(nb, generator=g)
    bt = torch.zeros(len(lens), max(max(pages), 1), dtype=torch.int32)
    slots = torch.empty(total, dtype=torch.int64)
    at, pg = 0, 0
    for b, n in enumerate(lens):
        ids = perm[pg:pg + pages[b]]
        bt[b, :pages[b]] = ids.to(torch.int32)
        t = torch.arange(n)
        slots[at:at + n] = ids[t // 16] * 16 + t % 16
        at += n
        pg += pages[b]
    q = torch.randn(len(lens), Hq, d, generator=g).to(dtype)
    return k, v, q, bt, slots, nb


@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (128, torch.float16), (128, torch.float32),
                                     (64, torch.bfloat16), (256, torch.float16)])
def test_store_bytes_equal_the_oracle(d, dtype):
    lens = [40, 0, 333, 16]
    k, v, q, bt, slots, nb = _case(3 + d, lens, 2, 8, d, dtype)
    slots[7] = -1
    v[11] = 1.25                                           # a constant row
    sb = _cabi.nc_slot_bytes(d)
    want = np.full((nb, 16, 2, sb), 0x5A, np.uint8)
    tq_oracle.nc_store(want, k.float().numpy(), v.float().numpy(), slots.numpy())
    cache = torch.full((nb, 16, 2, sb), 0x5A, dtype=torch.uint8, device=DEV)
    _cabi.nc_write_kv_cache(k.to(DEV), v.to(DEV), cache, slots.to(DEV))
    torch.cuda.synchronize()
    got = cache.cpu().numpy()
    diff = np.argwhere(got != want)
    assert len(diff) == 0, f"{len(diff)} bytes differ, first at (page, entry, head, byte) {diff[0].tolist()}: " \
                           f"{int(got[tuple(diff[0])])} vs {int(want[tuple(diff[0])])}; bytes of the slot that differ: " \
                           f"{sorted(set(int(x[3]) for x in diff if (x[:3] == diff[0][:3]).all()))}"
    # int32 slots and a slot id outside the cache: skipped and counted
    before = _cabi.nc_write_dropped()
    bad = slots.to(torch.int32).clone()
    bad[0] = nb * 16 + 5
    cache2 = torch.full_like(cache, 0x5A)
    _cabi.nc_write_kv_cache(k.to(DEV), v.to(DEV), cache2, bad.to(DEV))
    torch.cuda.synchronize()
    assert _cabi.nc_write_dropped() == before + 1
    want2 = want.copy()
    want2.reshape(-1, 2, sb)[int(slots[0])] = 0x5A
    assert np.array_equal(cache2.cpu().numpy(), want2)


@pytest.mark.parametrize("d,Hq,H,dtype", [(128, 32, 8, torch.bfloat16), (128, 8, 8, torch.float16), (64, 16, 2, torch.bfloat16),
                                          (256, 8, 4, torch.float16)])
def test_decode_matches_the_oracle(d, Hq, H, dtype):
    lens = [40, 0, 1000, 16, 2100, 1]
    k, v, q, bt, slots, nb = _case(17 + d + Hq, lens, H, Hq, d, dtype)
    sb = _cabi.nc_slot_bytes(d)
    cache = torch.zeros((nb, 16, H, sb), dtype=torch.uint8, device=DEV)
    _cabi.nc_write_kv_cache(k.to(DEV), v.to(DEV), cache, slots.to(DEV))
    sl = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    want, want_lse = tq_oracle.nc_decode(q.float().numpy(), cache.cpu().numpy(), bt.numpy(), lens, scale, return_lse=True)
    for ctas in (0, 3):
        ws = torch.zeros(_cabi.nc_decode_workspace_bytes(len(lens), Hq, H, d, ctas), dtype=torch.uint8, device=DEV)
        out = torch.full_like(q, float("nan"), device=DEV)
        lse = torch.empty(len(lens), Hq, dtype=torch.float32, device=DEV)
        _cabi.nc_decode_paged(q.to(DEV), cache, bt.to(DEV), sl.to(DEV), scale, ws, out, out_lse=lse, num_ctas=ctas)
        torch.cuda.synchronize()
        assert ws[:4].view(torch.int32).item() == 0
        got = out.float().cpu().numpy()
        err = np.abs(got - want)
        assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), err.max()
        assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-2
        assert (got[1] == 0).all()
        ok = np.isfinite(want_lse)
        np.testing.assert_allclose(lse.cpu().numpy()[ok], want_lse[ok], atol=2e-3)


def test_bad_ids_are_reported_not_followed():
    k, v, q, bt, slots, nb = _case(5, [100], 8, 32, 128, torch.bfloat16)
    cache = torch.zeros((nb, 16, 8, 134), dtype=torch.uint8, device=DEV)
    _cabi.nc_write_kv_cache(k.to(DEV), v.to(DEV), cache, slots.to(DEV))
    ws = torch.zeros(_cabi.nc_decode_workspace_bytes(1, 32, 8, 128), dtype=torch.uint8, device=DEV)
    out = torch.empty_like(q, device=DEV)
    bad = bt.clone()
    bad[0, 2] = nb + 1000
    _cabi.nc_decode_paged(q.to(DEV), cache, bad.to(DEV), torch.tensor([100], dtype=torch.int32, device=DEV), 128 ** -0.5, ws, out)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 5
    ws.zero_()
    _cabi.nc_decode_paged(q.to(DEV), cache, bt.to(DEV), torch.tensor([100 + 16 * bt.shape[1]], dtype=torch.int32, device=DEV),
                          128 ** -0.5, ws, out)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 4
    with pytest.raises(_cabi.TurboQuantError, match="head_dim"):
        _cabi.nc_slot_bytes(96)
