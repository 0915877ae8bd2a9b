"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

Everything is drawn from ``torch.Generator("cpu").manual_seed(seed)`` in fp32 and then cast,
so the same inputs can be rebuilt on any machine.  These stand in for the serving traces
the reference benchmarks with; no dataset item is reproduced here.

Geometry shared by all configs: 32 query heads, 8 KV heads (GQA group 4), head_dim 128,
16-token pages, 80-byte cache slots (turboquant/vllm_backend_fused.py:57-86 in the reference).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

NUM_Q_HEADS = 32
NUM_KV_HEADS = 8
HEAD_DIM = 128
PAGE = 16
SLOT_BYTES = 80


def make_signs(padded_dim: int = 128, seed: int = 42) -> torch.Tensor:
    """The reference's sign recipe (turboquant/hadamard.py:52-60): sign(randn) with 0 -> +1."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    signs = torch.sign(torch.randn(padded_dim, generator=gen))
    signs[signs == 0] = 1.0
    return signs


@dataclass
class DecodeCase:
    q: torch.Tensor             # [B, Hq, D]
    k: torch.Tensor             # [sum(len), H, D]  tokens of all sequences, concatenated
    v: torch.Tensor
    seq_lens: torch.Tensor      # [B] int32
    block_table: torch.Tensor   # [B, max_pages] int32
    slot_mapping: torch.Tensor  # [sum(len)] int64
    num_blocks: int


def paged_layout(seq_lens, seed: int | None, page: int = PAGE, extra_blocks: int = 0):
    """Block table + slot mapping for sequences laid into a (seeded) permutation of pages.
    ``seed=None`` gives the identity block table."""
    seq_lens = [int(x) for x in seq_lens]
    pages = [(n + page - 1) // page for n in seq_lens]
    total = sum(pages)
    num_blocks = total + extra_blocks
    if seed is None:
        perm = torch.arange(num_blocks, dtype=torch.int64)
    else:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        perm = torch.randperm(num_blocks, generator=gen)
    max_pages = max(pages) if pages else 0
    block_table = torch.zeros((len(seq_lens), max(max_pages, 1)), dtype=torch.int32)
    slots = []
    at = 0
    for b, (n, p) in enumerate(zip(seq_lens, pages)):
        ids = perm[at:at + p]
        at += p
        block_table[b, :p] = ids.to(torch.int32)
        t = torch.arange(n, dtype=torch.int64)
        slots.append(ids[t // page] * page + t % page)
    slot_mapping = torch.cat(slots) if slots else torch.zeros(0, dtype=torch.int64)
    return block_table, slot_mapping, num_blocks


def decode_case(seed: int, seq_lens, dtype=torch.float16, permute_pages: bool = True,
                num_q_rows: int | None = None, heads=(NUM_Q_HEADS, NUM_KV_HEADS),
                head_dim: int = HEAD_DIM) -> DecodeCase:
    """Q, K, V i.i.d. N(0,1) from ``seed``; pages permuted with the same seed unless told not to."""
    hq, hkv = heads
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    B = len(seq_lens) if num_q_rows is None else num_q_rows
    total = int(sum(int(x) for x in seq_lens))
    q = torch.randn(B, hq, head_dim, generator=gen).to(dtype)
    k = torch.randn(total, hkv, head_dim, generator=gen).to(dtype)
    v = torch.randn(total, hkv, head_dim, generator=gen).to(dtype)
    bt, slots, nb = paged_layout(seq_lens, seed if permute_pages else None)
    return DecodeCase(q, k, v, torch.tensor([int(x) for x in seq_lens], dtype=torch.int32), bt,
                      slots, nb)


def write_case(seed: int = 2, num_tokens: int = 32768, dtype=torch.bfloat16,
               outlier_frac: float = 0.01, outlier_scale: float = 20.0, num_skipped: int = 0):
    """Cache-write workload: K ~ N(0,1) with round(frac*128) channels scaled, V ~ N(0,1);
    tokens scattered into a seeded permutation of 16-token pages; ``num_skipped`` slots = -1."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    k = torch.randn(num_tokens, NUM_KV_HEADS, HEAD_DIM, generator=gen)
    v = torch.randn(num_tokens, NUM_KV_HEADS, HEAD_DIM, generator=gen)
    n_out = max(1, int(round(outlier_frac * HEAD_DIM))) if outlier_frac > 0 else 0
    chans = torch.randperm(HEAD_DIM, generator=gen)[:n_out]
    k[..., chans] *= outlier_scale
    _, slots, nb = paged_layout([num_tokens], seed)
    if num_skipped:
        skip = torch.randperm(num_tokens, generator=gen)[:num_skipped]
        slots[skip] = -1
    return k.to(dtype), v.to(dtype), slots, nb


def mixed_lengths(seed: int = 3, n: int = 64, lo: int = 512, hi: int = 131072):
    """Lengths floor(exp(U(ln lo, ln hi))) (the mixed-length decode config)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    u = torch.rand(n, generator=gen, dtype=torch.float64)
    return [int(math.floor(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo)))))
            for x in u]
