"""Helpers shared by the GPU parity tests: build caches with the oracle, run the CUDA path."""
import math

import numpy as np
import torch

from turboquant_b200 import _cabi, synthetic

DEV = "cuda"


def signs_dev():
    return synthetic.make_signs(128, 42).to(DEV)


def oracle_cache(oracle, case, signs_np):
    H = case.k.shape[1]
    cache = np.zeros((2, case.num_blocks, 16, H, 80), np.uint8)
    oracle.write_kv_cache(cache, case.k.float().numpy(), case.v.float().numpy(), signs_np,
                          case.slot_mapping.numpy(), 128)
    return cache


def run_decode(q, cache_dev, block_table, seq_lens, sm_scale=None, out_dtype=None, num_ctas=0,
               page_indptr=None, want_lse=False):
    B, Hq, D = q.shape
    H = cache_dev.shape[3]
    sm_scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    ws = torch.zeros(_cabi.decode_workspace_bytes(B, Hq, H, D, num_ctas), dtype=torch.uint8, device=DEV)
    out = torch.empty(B, Hq, D, dtype=out_dtype or q.dtype, device=DEV)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=DEV) if want_lse else None
    _cabi.decode_paged(q, cache_dev, block_table, seq_lens, signs_dev(), sm_scale, ws, out,
                       page_indptr=page_indptr, out_lse=lse, num_ctas=num_ctas,
                       max_pages=block_table.shape[-1] if block_table.dim() == 2 else 1)
    torch.cuda.synchronize()
    status = ws[:4].view(torch.int32).item()
    assert status == 0, f"decode kernel status {status}"
    return (out, lse) if want_lse else out


def assert_attention_close(got, want, what="", strict=False):
    """Parity bar for attention outputs against the dequant-attention oracle.

    Mixed bar (always): every element within max-abs 2e-3 + relative 1e-2 of the oracle value
    (an fp16/bf16 output of magnitude ~1 cannot be closer than its own rounding step, 1.95e-3
    for bf16), and the whole tensor within 1e-2 relative error in the Frobenius norm.
    ``strict`` additionally asserts the plain reading of the bar, max-abs <= 2e-3 AND relative
    <= 1e-2; it holds wherever the outputs are well below 1 (the long-context configs) or the
    output type is fp32/fp16.  Returns (max-abs, relative) so that callers can record them."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    bound = 2e-3 + 1e-2 * np.abs(want)
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    worst = (err - bound).max()
    assert worst <= 0, f"{what}: element error {err.max():.3e} exceeds 2e-3 + 1e-2*|ref| by {worst:.3e} (rel {rel:.3e})"
    assert rel <= 1e-2, f"{what}: relative {rel:.3e} > 1e-2 (max-abs {err.max():.3e})"
    if strict:
        assert err.max() <= 2e-3, f"{what}: strict max-abs {err.max():.3e} > 2e-3 (rel {rel:.3e})"
    return err.max(), rel


def fill_cache_gpu(cache, block_table_row, n_tokens, gen, chunk=65536, heads=8):
    """Seeded N(0,1) bf16 K/V for one sequence, quantized into its pages by the CUDA write kernel
    (bit-identical to the oracle's write, which the write tests establish)."""
    signs = signs_dev()
    for t0 in range(0, n_tokens, chunk):
        n = min(chunk, n_tokens - t0)
        k = torch.randn(n, heads, 128, generator=gen, device=DEV).to(torch.bfloat16)
        v = torch.randn(n, heads, 128, generator=gen, device=DEV).to(torch.bfloat16)
        tok = torch.arange(t0, t0 + n, device=DEV)
        slots = block_table_row.long()[tok // 16] * 16 + tok % 16
        _cabi.write_kv_cache(cache, k, v, signs, slots, 128)
