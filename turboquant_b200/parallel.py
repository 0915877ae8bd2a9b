"""Multi-GPU helpers (one process per GPU, ``torch.distributed``).

Two ways the decode path shards:

* by sequence (``shard_sequences``): attention is independent per sequence, every rank decodes its
  own sequences with no communication;
* along the KV axis of one long sequence (``kv_split_decode``): rank r holds the pages of a
  contiguous token range, computes the normalized rotated-domain partial and its base-2 LSE with
  ``tq_decode_paged_partial``, the partials are all-gathered (132 KB per rank at 8 queries x 32
  heads) and every rank finishes with the LSE merge + inverse rotation (``tq_merge_rotated``).

``merge_gathered`` is the collective-free core of the second path and is what the CPU (gloo)
tests exercise with oracle-made partials.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_sequences(seq_lens, world_size: int):
    """Greedy longest-first assignment of sequences to ranks; returns a list of index lists whose
    total lengths are balanced (max/mean reported by the caller)."""
    order = sorted(range(len(seq_lens)), key=lambda i: -int(seq_lens[i]))
    loads = [0] * world_size
    shards = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: loads[j])
        shards[r].append(i)
        loads[r] += int(seq_lens[i])
    return [sorted(s) for s in shards]


def kv_ranges(total_tokens: int, world_size: int, page: int = 16):
    """Contiguous, page-aligned token ranges [begin, end) per rank."""
    pages = (total_tokens + page - 1) // page
    out = []
    for r in range(world_size):
        p0, p1 = (pages * r) // world_size, (pages * (r + 1)) // world_size
        out.append((p0 * page, min(p1 * page, total_tokens)))
    return out


def all_gather_partials(part_o: torch.Tensor, part_lse2: torch.Tensor, group=None):
    """[rows.., D], [rows..] on every rank -> ([world, rows.., D], [world, rows..])."""
    world = dist.get_world_size(group)
    part_o, part_lse2 = part_o.contiguous(), part_lse2.contiguous()
    # gathered along dim 0 (the layout every backend accepts), then viewed as [world, ...]
    o = torch.empty((world * part_o.shape[0],) + tuple(part_o.shape[1:]), dtype=part_o.dtype, device=part_o.device)
    l = torch.empty((world * part_lse2.shape[0],) + tuple(part_lse2.shape[1:]), dtype=part_lse2.dtype,
                    device=part_lse2.device)
    dist.all_gather_into_tensor(o, part_o, group=group)
    dist.all_gather_into_tensor(l, part_lse2, group=group)
    o = o.view((world,) + tuple(part_o.shape))
    l = l.view((world,) + tuple(part_lse2.shape))
    return o, l


def kv_split_decode(attn, query, kv_cache_local, block_table_local, seq_lens_local, output, group=None):
    """Decode ``query`` against a KV cache whose token axis is split over the ranks of ``group``.
    Every rank passes the part of the cache it holds (its own block table and local lengths).
    ``query`` is [rows, heads, D], or [rows, queries, heads, D] when the queries of a row share
    that row's KV (streamed once for all of them)."""
    from . import _cabi
    dev = query.device
    part_o = torch.empty(tuple(query.shape), dtype=torch.float32, device=dev)
    part_l = torch.empty(tuple(query.shape[:-1]), dtype=torch.float32, device=dev)
    if query.dim() == 4:
        _cabi.decode_paged_multi(query, attn._as_bytes(kv_cache_local), block_table_local, seq_lens_local,
                                 attn.signs(dev), attn.scale, attn.workspace(query.shape[0], dev, query.shape[1]),
                                 part_o, out_lse=part_l, rotated_partial=True)
    else:
        _cabi.decode_paged_partial(query, attn._as_bytes(kv_cache_local), block_table_local, seq_lens_local,
                                   attn.signs(dev), attn.scale, attn.workspace(query.shape[0], dev), part_o, part_l)
    o, l = all_gather_partials(part_o, part_l, group)
    _cabi.merge_rotated(o, l, attn.signs(dev), output)
    return output
