"""Generates the golden fixtures in this directory by running the REFERENCE's own Python
modules (imported from its source tree) on the CPU.  Run only where that tree exists:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [/path/to/reference]

The fixtures pin the CPU oracle (oracle/tq_oracle.c) and, through it, the CUDA kernels.
Nothing here is needed at test time; the .npz files are committed.
"""
import hashlib
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TURBOQUANT_REFERENCE", "")
if not REF:
    raise SystemExit("usage: make_golden.py <root of the reference tree>  (or set TURBOQUANT_REFERENCE)")
sys.path.insert(0, REF)
sys.path.insert(1, str(REPO))

from turboquant import Codebook, RandomHadamardRotation, TurboQuantMSE, fwht  # noqa: E402  (reference)
from turboquant.tile import pack_4bit, unpack_4bit  # noqa: E402  (reference)
from turboquant_b200 import synthetic  # noqa: E402

torch.set_num_threads(8)
CPU = "cpu"


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def ref_cache_write(k, v, slot_mapping, num_blocks, head_dim=128, page=16, ebs=80):
    """The reference quantizer on K and V, re-packed to the cache nibble order and scattered
    (BASELINE CPU path: TurboQuantMSE.quantize + tile.pack_4bit + scatter by slot)."""
    H = k.shape[1]
    tq = TurboQuantMSE(head_dim, 4, device=CPU, seed=42)
    cache = torch.zeros(2, num_blocks, page, H, ebs, dtype=torch.uint8)
    for i, x in enumerate((k, v)):
        packed_low, norms = tq.quantize(x.float())
        idx = torch.zeros(*packed_low.shape[:-1], head_dim, dtype=torch.uint8)
        idx[..., 0::2] = packed_low & 0x0F
        idx[..., 1::2] = packed_low >> 4
        packed = pack_4bit(idx)
        nh = norms.to(torch.float16).view(torch.uint8).reshape(*norms.shape, 2)
        slot = torch.cat([packed, nh, nh], dim=-1)          # 64 + 2 + 2 bytes
        ok = slot_mapping >= 0
        s = slot_mapping[ok]
        cache[i, s // page, s % page, :, :68] = slot[ok]
    return cache


def ref_dequant_attention(q, cache, block_table, seq_lens, scale, head_dim=128, page=16):
    """The reference dequant-attention path: unpack -> centroids -> inverse rotation -> x fp16
    norm -> fp32 softmax(q K^T scale) V (tests/test_fused_integration.py:127-159)."""
    tq = TurboQuantMSE(head_dim, 4, device=CPU, seed=42)
    B, Hq, D = q.shape
    H = cache.shape[3]
    out = torch.zeros(B, Hq, D)
    lse = torch.zeros(B, Hq)
    for b in range(B):
        n = int(seq_lens[b])
        t = torch.arange(n)
        pages = block_table[b, t // page].long()
        deq = []
        for i in range(2):
            slots = cache[i, pages, t % page]                # [n, H, ebs]
            idx = unpack_4bit(slots[..., :64], head_dim)
            y = tq.codebook.dequantize(idx)
            x = tq.rotation.inverse_rotate(y)
            norms = slots[..., 64:66].contiguous().view(torch.float16).float()
            deq.append(x * norms)
        kd, vd = deq
        g = Hq // H
        kd = kd.repeat_interleave(g, dim=1).transpose(0, 1)   # [Hq, n, D]
        vd = vd.repeat_interleave(g, dim=1).transpose(0, 1)
        s = torch.einsum("hd,hnd->hn", q[b].float(), kd) * scale
        lse[b] = torch.logsumexp(s, dim=-1)
        out[b] = torch.einsum("hn,hnd->hd", torch.softmax(s, dim=-1), vd)
    return out, lse


def main():
    fx = {}
    # ---- signs and codebooks -------------------------------------------------------------
    for dim in (64, 128, 256):
        fx[f"signs_seed42_d{dim}"] = RandomHadamardRotation(dim, CPU, seed=42).signs.numpy()
    fx["signs_seed7_d128"] = RandomHadamardRotation(128, CPU, seed=7).signs.numpy()
    fx["signs_seed42_d96"] = RandomHadamardRotation(96, CPU, seed=42).signs.numpy()
    for dim in (64, 128, 256):
        for bits in (1, 2, 3, 4):
            cb = Codebook(dim, bits, CPU)
            fx[f"centroids_d{dim}_b{bits}"] = cb.centroids.numpy()
            fx[f"boundaries_d{dim}_b{bits}"] = cb.boundaries.numpy()
    # ---- FWHT ----------------------------------------------------------------------------
    gen = torch.Generator(CPU).manual_seed(100)
    xf = torch.randn(16, 128, generator=gen)
    fx["fwht_in"] = xf.numpy()
    fx["fwht_out"] = fwht(xf).numpy()
    fx["fwht_kat_out"] = fwht(torch.tensor([1.0, 0, 0, 0])).numpy()
    # ---- quantizer rows: ordinary, outlier channel, bf16/fp16-sourced, degenerate ----------
    gen = torch.Generator(CPU).manual_seed(101)
    rows = torch.randn(768, 128, generator=gen)
    rows[128:256] = rows[128:256].to(torch.bfloat16).float()
    rows[256:384] = rows[256:384].to(torch.float16).float()
    rows[384:512, 77] *= 20.0                                   # outlier channel
    rows[384:512] = rows[384:512].to(torch.bfloat16).float()
    rows[512] = 0.0                                             # zero vector -> clamp path
    rows[513] = 0.0; rows[513, 5] = 1.0                          # one-hot: many exact ties in |y|
    rows[514] = 0.0; rows[514, 0] = 1.0; rows[514, 1] = 1.0      # exact zeros after the FWHT
    rows[515] = 0.0; rows[515, 3] = -2.5; rows[515, 64] = 2.5
    rows[516] = 1e-12 * rows[516]                                # below the clamp
    rows[517] = 1e4 * rows[517]
    rows[518] = 1.0                                              # constant vector
    rows[519] = torch.arange(128, dtype=torch.float32) - 63.5
    rows[520:640] *= torch.logspace(-6, 6, 120).unsqueeze(1)     # wide dynamic range
    rows[640, 3] = float("inf")                                  # inf element -> NaN spreads
    rows[641, 5] = float("nan")
    rows[642] = 1e30 * rows[642]                                 # sum of squares overflows
    rows[643] = 1e-30 * rows[643]                                # squares underflow to zero
    fx["q_rows"] = rows.numpy()
    tq = TurboQuantMSE(128, 4, CPU, seed=42)
    packed, norms = tq.quantize(rows)
    fx["q_packed_b4"] = packed.numpy()
    fx["q_norms"] = norms.numpy()
    fx["q_dequant_b4"] = tq.dequantize(packed[:64], norms[:64]).numpy()
    for bits in (1, 2, 3):
        tqb = TurboQuantMSE(128, bits, CPU, seed=42)
        p, n = tqb.quantize(rows[:128])
        fx[f"q_packed_b{bits}"] = p.numpy()
        fx[f"q_dequant_b{bits}"] = tqb.dequantize(p[:16], n[:16]).numpy()
    for dim in (64, 256, 96):
        gen = torch.Generator(CPU).manual_seed(102 + dim)
        r = torch.randn(96, dim, generator=gen).to(torch.bfloat16).float()
        tqd = TurboQuantMSE(dim, 4, CPU, seed=42)
        p, n = tqd.quantize(r)
        fx[f"q_rows_d{dim}"] = r.numpy()
        fx[f"q_packed_d{dim}"] = p.numpy()
        fx[f"q_norms_d{dim}"] = n.numpy()
    # nibble-order known answer (tests/test_tile.py:40-43 in the reference)
    fx["pack4_kat"] = pack_4bit(torch.tensor([0x0A, 0x05], dtype=torch.uint8)).numpy()
    # ---- small paged decode: ragged lengths, permuted pages ---------------------------------
    case = synthetic.decode_case(seed=11, seq_lens=[48, 21, 1], dtype=torch.float16)
    cache = ref_cache_write(case.k, case.v, case.slot_mapping, case.num_blocks)
    out, lse = ref_dequant_attention(case.q, cache, case.block_table, case.seq_lens,
                                     1.0 / math.sqrt(128))
    fx["att_q"] = case.q.numpy()
    fx["att_k"] = case.k.numpy()
    fx["att_v"] = case.v.numpy()
    fx["att_seq_lens"] = case.seq_lens.numpy()
    fx["att_block_table"] = case.block_table.numpy()
    fx["att_slot_mapping"] = case.slot_mapping.numpy()
    fx["att_cache"] = cache.numpy()
    fx["att_out"] = out.numpy()
    fx["att_lse"] = lse.numpy()
    # ---- config 0 in full: inputs by seed, pinned by hashes ---------------------------------
    c0 = synthetic.decode_case(seed=0, seq_lens=[1024], dtype=torch.float16, permute_pages=False)
    cache0 = ref_cache_write(c0.k, c0.v, c0.slot_mapping, c0.num_blocks)
    out0, lse0 = ref_dequant_attention(c0.q, cache0, c0.block_table, c0.seq_lens,
                                       1.0 / math.sqrt(128))
    fx["cfg0_out"] = out0.numpy()
    fx["cfg0_lse"] = lse0.numpy()
    fx["cfg0_sha_q"] = np.frombuffer(bytes.fromhex(sha(c0.q.view(torch.int16).numpy())), np.uint8)
    fx["cfg0_sha_k"] = np.frombuffer(bytes.fromhex(sha(c0.k.view(torch.int16).numpy())), np.uint8)
    fx["cfg0_sha_cache"] = np.frombuffer(bytes.fromhex(sha(cache0.numpy())), np.uint8)
    # ---- cache write with an outlier channel, bf16, skipped slots (config-2 recipe, 192 tokens)
    k2, v2, slots2, nb2 = synthetic.write_case(seed=2, num_tokens=192, num_skipped=7)
    cache2 = ref_cache_write(k2, v2, slots2, nb2)
    fx["wr_k_bf16_bits"] = k2.view(torch.int16).numpy()
    fx["wr_v_bf16_bits"] = v2.view(torch.int16).numpy()
    fx["wr_slots"] = slots2.numpy()
    fx["wr_cache"] = cache2.numpy()
    # config 2 in full: hash only (inputs by seed)
    k2f, v2f, slots2f, nb2f = synthetic.write_case(seed=2, num_tokens=32768, num_skipped=0)
    cache2f = ref_cache_write(k2f, v2f, slots2f, nb2f)
    fx["cfg2_sha_cache"] = np.frombuffer(bytes.fromhex(sha(cache2f.numpy())), np.uint8)
    fx["cfg2_sha_k"] = np.frombuffer(bytes.fromhex(sha(k2f.view(torch.int16).numpy())), np.uint8)
    np.savez_compressed(HERE / "golden.npz", **fx)
    total = sum(v.nbytes for v in fx.values())
    print(f"wrote {HERE / 'golden.npz'}: {len(fx)} arrays, {total / 1e6:.2f} MB raw, torch {torch.__version__}")


if __name__ == "__main__":
    main()
