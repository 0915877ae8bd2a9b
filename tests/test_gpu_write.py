"""Cache-write parity on the GPU: codes and fp16 norms bit-exact against the oracle and the
reference-generated fixtures, through the C ABI."""
import hashlib

import numpy as np
import pytest
import torch

from turboquant_b200 import _cabi, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def gpu_write(k, v, slots, nb, H=8, fill=0, zero_pad=False, signs=None):
    cache = torch.full((2, nb, 16, H, 80), fill, dtype=torch.uint8, device=DEV)
    signs = synthetic.make_signs(128, 42).to(DEV) if signs is None else signs
    _cabi.write_kv_cache(cache, k.to(DEV), v.to(DEV), signs, slots.to(DEV), 128, zero_pad=zero_pad)
    torch.cuda.synchronize()
    return cache.cpu().numpy()


def test_golden_write_case_bit_exact(golden):
    k = torch.from_numpy(golden["wr_k_bf16_bits"]).view(torch.bfloat16)
    v = torch.from_numpy(golden["wr_v_bf16_bits"]).view(torch.bfloat16)
    slots = torch.from_numpy(golden["wr_slots"])
    want = golden["wr_cache"]
    got = gpu_write(k, v, slots, want.shape[1])
    np.testing.assert_array_equal(got, want)
    # pad bytes and unmapped slots untouched
    got = gpu_write(k, v, slots, want.shape[1], fill=0xEE)
    assert (got[..., 68:] == 0xEE).all()
    written = np.zeros(want.shape[1] * 16, bool)
    written[golden["wr_slots"][golden["wr_slots"] >= 0]] = True
    flat = got.reshape(2, -1, 8, 80)
    assert (flat[:, ~written] == 0xEE).all()
    np.testing.assert_array_equal(flat[:, written][..., :68], want.reshape(2, -1, 8, 80)[:, written][..., :68])


def test_degenerate_rows_match_reference_quantizer(golden, oracle):
    """Zero / one-hot / tie / huge / tiny / inf / NaN rows from the reference fixture."""
    rows = torch.from_numpy(golden["q_rows"])                      # [768, 128] fp32
    k = rows.reshape(96, 8, 128)
    slots = torch.arange(96, dtype=torch.int64)
    got = gpu_write(k, k, slots, 6)
    codes = got[0].reshape(768, 80)[:, :64]
    want_codes = oracle.low_first_to_cache_order(golden["q_packed_b4"])
    np.testing.assert_array_equal(codes, want_codes)
    norms = got[0].reshape(768, 80)[:, 64:66].copy().view(np.float16).reshape(768)
    want = torch.from_numpy(golden["q_norms"]).to(torch.float16).numpy()
    np.testing.assert_array_equal(norms.view(np.uint16), want.view(np.uint16))
    np.testing.assert_array_equal(got[0], got[1])                  # V slab got the same rows
    np.testing.assert_array_equal(got[0].reshape(768, 80)[:, 66:68], got[0].reshape(768, 80)[:, 64:66])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_dtypes_vs_oracle(oracle, golden, dtype, slot_dtype):
    k, v, slots, nb = synthetic.write_case(seed=5, num_tokens=777, dtype=dtype, num_skipped=13)
    want = np.zeros((2, nb, 16, 8, 80), np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), golden["signs_seed42_d128"],
                          slots.numpy(), 128)
    got = gpu_write(k, v, slots.to(slot_dtype), nb)
    np.testing.assert_array_equal(got, want)


def test_strided_tokens_and_other_head_counts(oracle, golden):
    """key/value as column slices of a fused QKV activation; 4 and 1 KV heads."""
    for H in (4, 1, 2):
        gen = torch.Generator().manual_seed(H)
        T = 130
        qkv = torch.randn(T, (8 + 2 * H) * 128, generator=gen).to(torch.bfloat16)
        k = qkv[:, 8 * 128:(8 + H) * 128].unflatten(1, (H, 128))
        v = qkv[:, (8 + H) * 128:].unflatten(1, (H, 128))
        slots = torch.randperm(12 * 16, generator=gen)[:T]
        want = np.zeros((2, 12, 16, H, 80), np.uint8)
        oracle.write_kv_cache(want, k.float().contiguous().numpy(), v.float().contiguous().numpy(),
                              golden["signs_seed42_d128"], slots.numpy(), 128)
        qkv_d = qkv.to(DEV)
        kd = qkv_d[:, 8 * 128:(8 + H) * 128].unflatten(1, (H, 128))
        vd = qkv_d[:, (8 + H) * 128:].unflatten(1, (H, 128))
        cache = torch.zeros((2, 12, 16, H, 80), dtype=torch.uint8, device=DEV)
        _cabi.write_kv_cache(cache, kd, vd, synthetic.make_signs().to(DEV), slots.to(DEV), 128)
        np.testing.assert_array_equal(cache.cpu().numpy(), want)


def test_zero_pad_flag_and_empty_input(oracle, golden):
    k, v, slots, nb = synthetic.write_case(seed=6, num_tokens=64)
    got = gpu_write(k, v, slots, nb, fill=0xEE, zero_pad=True)
    assert (got[..., 68:] == 0).all()
    want = np.zeros((2, nb, 16, 8, 80), np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), golden["signs_seed42_d128"], slots.numpy(), 128)
    np.testing.assert_array_equal(got[..., :68], want[..., :68])
    cache = torch.zeros((2, 2, 16, 8, 80), dtype=torch.uint8, device=DEV)
    _cabi.write_kv_cache(cache, k[:0].to(DEV), v[:0].to(DEV), synthetic.make_signs().to(DEV),
                         slots[:0].to(DEV), 128)
    assert int(cache.sum()) == 0


def test_other_sign_seed(oracle, golden):
    k, v, slots, nb = synthetic.write_case(seed=8, num_tokens=100)
    signs = synthetic.make_signs(128, 7)
    want = np.zeros((2, nb, 16, 8, 80), np.uint8)
    oracle.write_kv_cache(want, k.float().numpy(), v.float().numpy(), signs.numpy(), slots.numpy(), 128)
    np.testing.assert_array_equal(gpu_write(k, v, slots, nb, signs=signs.to(DEV)), want)


def test_config2_full_size_checksum(golden):
    """32768 tokens x 8 heads, bf16, outlier channel, permuted pages: every byte equals the
    reference quantizer's (compared through a SHA-256 committed with the fixtures)."""
    k, v, slots, nb = synthetic.write_case(seed=2, num_tokens=32768)
    got = gpu_write(k, v, slots, nb)
    np.testing.assert_array_equal(sha(got), golden["cfg2_sha_cache"])


def test_flat_quantizer_api(golden):
    signs = synthetic.make_signs(128, 42).to(DEV)
    rows = torch.from_numpy(golden["q_rows"]).to(DEV)
    packed, norms = _cabi.quantize_flat(rows, signs, 4)
    np.testing.assert_array_equal(packed.cpu().numpy(), golden["q_packed_b4"])
    np.testing.assert_array_equal(norms.cpu().numpy().view(np.uint32), golden["q_norms"].view(np.uint32))
    for bits in (1, 2, 3):
        p, _ = _cabi.quantize_flat(rows[:128], signs, bits)
        np.testing.assert_array_equal(p.cpu().numpy(), golden[f"q_packed_b{bits}"])
        deq = _cabi.dequantize_flat(p[:16], norms[:16], signs, 128, bits)
        np.testing.assert_allclose(deq.cpu().numpy(), golden[f"q_dequant_b{bits}"], rtol=1e-5, atol=1e-30)
    deq = _cabi.dequantize_flat(packed[:64], norms[:64], signs, 128, 4)
    np.testing.assert_allclose(deq.cpu().numpy(), golden["q_dequant_b4"], rtol=1e-5, atol=1e-30)
    for dim in (64, 256, 96):
        pd = 1 << (dim - 1).bit_length()
        s = torch.from_numpy(golden[f"signs_seed42_d{dim}"]).to(DEV)
        assert s.numel() == pd
        p, n = _cabi.quantize_flat(torch.from_numpy(golden[f"q_rows_d{dim}"]).to(DEV), s, 4)
        np.testing.assert_array_equal(p.cpu().numpy(), golden[f"q_packed_d{dim}"])
        np.testing.assert_array_equal(n.cpu().numpy().view(np.uint32), golden[f"q_norms_d{dim}"].view(np.uint32))


def test_fwht_api(golden):
    x = torch.from_numpy(golden["fwht_in"]).to(DEV)
    np.testing.assert_array_equal(_cabi.fwht(x, 128, 128).cpu().numpy(), golden["fwht_out"])
    kat = _cabi.fwht(torch.tensor([1.0, 0, 0, 0], device=DEV), 4, 4)
    np.testing.assert_array_equal(kat.cpu().numpy(), np.full(4, 0.5, np.float32))
