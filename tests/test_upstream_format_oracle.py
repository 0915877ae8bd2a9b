"""CPU checks of the oracle's restatement of the upstream vLLM slot format ("turboquant_4bit_nc").
The reference tree describes the format (docs/reference/vllm-upstream-turboquant-architecture.md:33-175)
but holds no code or vectors for it, so these are consistency checks, not golden vectors."""
import numpy as np
import pytest

from oracle import tq_oracle


@pytest.mark.parametrize("d", [64, 128, 256])
def test_slot_layout_and_round_trip(d):
    rng = np.random.default_rng(d)
    T, H = 24, 2
    k = rng.standard_normal((T, H, d)).astype(np.float32)
    v = (rng.standard_normal((T, H, d)) * 3 + 1).astype(np.float32)
    sb = tq_oracle.nc_slot_bytes(d)
    assert sb == d + 6 and (d != 128 or sb == 134)
    cache = np.full((2, 16, H, sb), 0xAA, np.uint8)
    slots = np.arange(T)
    slots[5] = -1
    tq_oracle.nc_store(cache, k, v, slots)
    flat = cache.reshape(32, H, sb)
    assert (flat[5] == 0xAA).all() and (flat[T:] == 0xAA).all()
    qb, kps = d // 2, d // 2 + 2
    cen, _ = tq_oracle.codebook(d, 4)
    for t in (0, 7, T - 1):
        for h in range(H):
            s = flat[t, h]
            # V: code * scale + zero reproduces v within half a step; extremes map to codes 0 and 15
            vidx = np.stack((s[kps:kps + qb] & 15, s[kps:kps + qb] >> 4), -1).reshape(d)
            scale, zero = s[kps + qb:kps + qb + 4].copy().view(np.float16).astype(np.float32)
            assert vidx[np.argmin(v[t, h])] == 0 and vidx[np.argmax(v[t, h])] == 15
            assert np.abs(vidx * scale + zero - v[t, h]).max() <= 0.5 * scale + 2e-2
            # K: the norm is the row's L2 norm (fp16), the codes dequantize to a vector close to k
            kn = float(s[qb:qb + 2].copy().view(np.float16)[0])
            assert abs(kn - np.linalg.norm(k[t, h])) <= 1e-3 * kn
            kidx = np.stack((s[:qb] & 15, s[:qb] >> 4), -1).reshape(d)
            khat = tq_oracle.fwht(cen[kidx] * kn)          # the Hadamard matrix is its own inverse
            cos = float(khat @ k[t, h] / (np.linalg.norm(khat) * np.linalg.norm(k[t, h])))
            assert cos > 0.98


def test_constant_value_row_and_decode_against_plain_attention():
    rng = np.random.default_rng(1)
    T, H, d = 300, 2, 128
    k = rng.standard_normal((T, H, d)).astype(np.float32)
    v = rng.standard_normal((T, H, d)).astype(np.float32)
    v[3] = 2.5                                             # a constant row: scale 0, every code 0
    cache = np.zeros((19, 16, H, 134), np.uint8)
    tq_oracle.nc_store(cache, k, v, np.arange(T))
    s = cache.reshape(-1, H, 134)[3, 0]
    assert (s[66:130] == 0).all() and s[130:132].copy().view(np.float16)[0] == 0 and s[132:134].copy().view(np.float16)[0] == 2.5
    q = rng.standard_normal((1, 8, d)).astype(np.float32)
    bt = np.arange(19)[None]
    out, lse = tq_oracle.nc_decode(q, cache, bt, [T], d ** -0.5, return_lse=True)
    sc = np.einsum("hgd,nhd->hgn", q[0].reshape(H, 4, d), k) * d ** -0.5
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ref = np.einsum("hgn,nhd->hgd", p, v).reshape(8, d)
    assert np.linalg.norm(out[0] - ref) / np.linalg.norm(ref) < 0.35      # 4-bit K and V: same order as the project's own format
    assert np.isfinite(lse).all()
    empty = tq_oracle.nc_decode(q, cache, bt, [0], d ** -0.5)
    assert (empty == 0).all()
