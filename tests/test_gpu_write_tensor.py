"""The tensor-core cache-write kernel (large fp16 / bf16 writes) against the kernel that evaluates
the reference's arithmetic for every element, and against the oracle: every byte must be equal.

The fast kernel takes a code from its own transform only when the value is farther than 2^-18
from the bin's boundary and re-derives the rest exactly, so the cases here aim at what could
break that: degenerate rows, values engineered to sit next to every boundary, and volume."""
import math

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"


def write(k, v, slots, nb, path, H=8, fill=0):
    cache = torch.full((2, nb, 16, H, 80), fill, dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, k, v, synthetic.make_signs(128, 42).to(DEV), slots, 128, path=path)
    return cache


def test_degenerate_rows_through_the_tensor_kernel(golden, oracle):
    """The reference fixture's zero / one-hot / tie / tiny / huge / inf / NaN rows, rounded to bf16
    and fp16 so that the tensor kernel accepts them: bytes equal the exact kernel's and the oracle's."""
    rows = torch.from_numpy(golden["q_rows"])                       # [768, 128] fp32
    for dtype in (torch.bfloat16, torch.float16):
        k = rows.to(dtype).reshape(96, 8, 128)
        slots = torch.arange(96, dtype=torch.int64)
        exact = write(k.to(DEV), k.to(DEV), slots.to(DEV), 6, "exact").cpu().numpy()
        fast = write(k.to(DEV), k.to(DEV), slots.to(DEV), 6, "tensor").cpu().numpy()
        np.testing.assert_array_equal(fast, exact)
        want = np.zeros((2, 6, 16, 8, 80), np.uint8)
        oracle.write_kv_cache(want, k.float().numpy(), k.float().numpy(), golden["signs_seed42_d128"], slots.numpy(), 128)
        # Codes everywhere; norms wherever they are numbers.  Which NaN pattern a NaN input leaves in
        # the norm (sign, payload) is a property of the host's arithmetic, not of the quantizer: the
        # kernels store the canonical quiet NaN there.
        got_n = fast.reshape(2, 768, 80)[:, :, 64:68].copy().view(np.float16)
        want_n = want.reshape(2, 768, 80)[:, :, 64:68].copy().view(np.float16)
        nan = np.isnan(want_n)
        assert nan.any() and np.isnan(got_n[nan]).all()
        np.testing.assert_array_equal(got_n[~nan].view(np.uint16), want_n[~nan].view(np.uint16))
        np.testing.assert_array_equal(fast[..., :64], want[..., :64])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_small_and_ragged_writes_vs_oracle(oracle, golden, dtype):
    for T, H, skipped in ((1, 8, 0), (37, 8, 3), (777, 8, 13), (130, 4, 0), (65, 1, 2), (200, 5, 0)):
        gen = torch.Generator().manual_seed(T + H)
        k = torch.randn(T, H, 128, generator=gen).to(dtype)
        v = (torch.randn(T, H, 128, generator=gen) * 3.0).to(dtype)
        nb = (T + 15) // 16 + 2
        slots = torch.randperm(nb * 16, generator=gen)[:T]
        if skipped:
            slots[torch.randperm(T, generator=gen)[:skipped]] = -1
        want = np.full((2, nb, 16, H, 80), 0xEE, np.uint8)
        oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), golden["signs_seed42_d128"], slots.numpy(), 128)
        got = write(k.to(DEV), v.to(DEV), slots.to(DEV), nb, "tensor", H=H, fill=0xEE).cpu().numpy()
        np.testing.assert_array_equal(got, want)


def test_strided_qkv_and_int32_slots(oracle, golden):
    gen = torch.Generator().manual_seed(3)
    T, H = 600, 8
    qkv = torch.randn(T, (32 + 2 * H) * 128, generator=gen).to(torch.bfloat16)
    k = qkv[:, 32 * 128:(32 + H) * 128].unflatten(1, (H, 128))
    v = qkv[:, (32 + H) * 128:].unflatten(1, (H, 128))
    slots = torch.randperm(40 * 16, generator=gen)[:T].to(torch.int32)
    want = np.zeros((2, 40, 16, H, 80), np.uint8)
    oracle.write_kv_cache(want, k.float().contiguous().numpy(), v.float().contiguous().numpy(),
                          golden["signs_seed42_d128"], slots.numpy(), 128)
    qd = qkv.to(DEV)
    got = write(qd[:, 32 * 128:(32 + H) * 128].unflatten(1, (H, 128)), qd[:, (32 + H) * 128:].unflatten(1, (H, 128)),
                slots.to(DEV), 40, "tensor")
    np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_config2_full_size_checksum_both_paths(golden):
    import hashlib
    k, v, slots, nb = synthetic.write_case(seed=2, num_tokens=32768)
    for path in ("tensor", "exact", "auto"):
        got = write(k.to(DEV), v.to(DEV), slots.to(DEV), nb, path).cpu().numpy()
        digest = np.frombuffer(hashlib.sha256(np.ascontiguousarray(got).tobytes()).digest(), np.uint8)
        np.testing.assert_array_equal(digest, golden["cfg2_sha_cache"], err_msg=path)


def _near_boundary_pairs(bnd, per_boundary=64):
    """bf16 amplitude pairs (a, b) such that a two-hot row has |y| = (a + b) / (sqrt(a^2 + b^2) sqrt(128))
    or (a - b) / ... within a few 1e-6 of a code boundary."""
    a = torch.arange(0x3F80, 0x4000, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).double()   # [1, 2)
    ratios = []
    for e in range(0, 9):
        ratios.append(a / (2.0 ** e))
    b_all = torch.cat(ratios)                                   # candidates for the smaller amplitude
    A, B = torch.meshgrid(a, b_all, indexing="ij")
    n = torch.sqrt(A * A + B * B) * math.sqrt(128.0)
    found = []
    for y in ((A + B) / n, (A - B) / n):
        for bd in bnd:
            if bd <= 0:
                continue
            d = (y - float(bd)).abs().flatten()
            idx = torch.topk(-d, per_boundary).indices
            keep = idx[d[idx] < 1.6e-5]
            found.append(torch.stack([A.flatten()[keep], B.flatten()[keep]], 1))
    return torch.cat(found)


def test_values_engineered_next_to_every_boundary(oracle):
    """Two-hot rows whose transformed values all sit within about 4 x the guard distance of a code
    boundary (amplitude pairs searched on the host), in random positions and with random signs:
    more than 1e8 such elements, tensor kernel against exact kernel, and a sample against the oracle."""
    _, bnd = oracle.codebook(128, 4)
    pairs = _near_boundary_pairs(torch.from_numpy(bnd).double())
    assert pairs.shape[0] >= 100
    gen = torch.Generator().manual_seed(9)
    rows = 1 << 21                                              # 2M rows x 128 values, at least 64 near a boundary
    pick = torch.randint(0, pairs.shape[0], (rows,), generator=gen)
    pos = torch.rand(rows, 128, generator=gen).argsort(1)[:, :2]
    sgn = torch.randint(0, 2, (rows, 2), generator=gen).double() * 2 - 1
    x = torch.zeros(rows, 128, dtype=torch.bfloat16)
    scale = torch.exp2(torch.randint(-6, 7, (rows, 1), generator=gen).double())
    amp = pairs[pick] * sgn * scale
    x.scatter_(1, pos, amp.to(torch.bfloat16))
    k = x.view(rows // 8, 8, 128).to(DEV)
    T = rows // 8
    nb = T // 16
    slots = torch.randperm(T, generator=gen).to(DEV)
    before = _cabi.write_guard_stats()
    fast = write(k, k, slots, nb, "tensor")
    exact = write(k, k, slots, nb, "exact")
    assert torch.equal(fast, exact)
    after = _cabi.write_guard_stats()
    assert after[1] - before[1] > 0.1 * (after[0] - before[0])   # the guard did trigger on these rows
    sample = slice(0, 4096)
    want = np.zeros((2, nb, 16, 8, 80), np.uint8)
    sl = slots.cpu().numpy().copy()
    sl[4096:] = -1
    oracle.write_kv_cache(want, k.float().cpu().numpy(), k.float().cpu().numpy(), synthetic.make_signs().numpy(), sl, 128)
    got = fast.cpu().numpy().reshape(2, -1, 8, 80)
    idx = sl[sample]
    np.testing.assert_array_equal(got[:, idx], want.reshape(2, -1, 8, 80)[:, idx])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_volume_random_rows(dtype):
    """5e8 random elements (N(0,1), a x20 outlier channel, a few scaled rows): tensor kernel ==
    exact kernel byte for byte; the share of rows re-derived exactly is reported and bounded."""
    gen = torch.Generator(device=DEV)
    gen.manual_seed(11)
    T = 1 << 18
    nb = T // 16
    slots = torch.randperm(T, generator=torch.Generator().manual_seed(1)).to(DEV)
    flagged = total = 0
    for rep in range(2):
        k = torch.randn(T, 8, 128, generator=gen, device=DEV)
        v = torch.randn(T, 8, 128, generator=gen, device=DEV)
        k[..., 17] *= 20.0
        v[::5] *= 1e-3
        v[::7] *= 300.0
        k, v = k.to(dtype), v.to(dtype)
        before = _cabi.write_guard_stats()
        fast = write(k, v, slots, nb, "tensor")
        exact = write(k, v, slots, nb, "exact")
        assert torch.equal(fast, exact), f"rep {rep}: {(fast != exact).sum().item()} bytes differ"
        after = _cabi.write_guard_stats()
        total += after[0] - before[0]
        flagged += after[1] - before[1]
    share = flagged / total
    print(f"{dtype}: {total} rows, {flagged} re-derived exactly ({100 * share:.2f} %)")
    assert 0.005 < share < 0.08
