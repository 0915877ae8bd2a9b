"""Multi-GPU helpers (one process per GPU, ``torch.distributed``).

Two ways the decode path shards:

* by sequence (``shard_sequences``): attention is independent per sequence, every rank decodes its
  own sequences with no communication;
* along the KV axis of one long sequence (``kv_split_decode``): rank r holds the pages of a
  contiguous token range, computes the normalized rotated-domain partial and its base-2 LSE with
  ``tq_decode_paged_partial``, the partials are all-gathered (132 KB per rank at 8 queries x 32
  heads) and every rank finishes with the LSE merge + inverse rotation (``tq_merge_rotated``).

``KVSplitExchange`` is the fused form of the second path: the decode's merge epilogue stores the
partial straight into every rank's exchange buffer over NVLink and a flag-gated merge finishes,
so no collective library call sits between the two kernels.

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
    # rotated partials are as wide as the padded head (96 -> 128, 80 -> 128, 192 -> 256)
    part_o = torch.empty(tuple(query.shape[:-1]) + (attn.padded_dim,), dtype=torch.float32, device=dev)
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


class KVSplitExchange:
    """KV-axis split decode whose exchange is done by the kernels themselves
    (``tq_decode_paged_exchange``): plain peer stores into every rank's buffer, a per-source flag,
    a bounded wait, then the LSE merge and the inverse rotation on every rank.

    The buffers are symmetric memory (``torch.distributed._symmetric_memory``), zeroed and
    rendezvoused once here; ``decode`` itself allocates nothing and can be graph-captured.
    Multicast (NVLS) binding of the buffer is switched off: the kernels use plain peer stores only.
    """

    def __init__(self, attn, batch: int, queries: int, device, group=None, buffers=None):
        from . import _cabi
        self.attn = attn
        self.batch, self.queries = batch, queries
        self.group = group
        self.world = dist.get_world_size(group) if buffers is None else len(buffers)
        self.rank = dist.get_rank(group) if buffers is None else 0
        rows = batch * queries * attn.num_heads
        self.nbytes = _cabi.exchange_bytes(rows, self.world)
        if buffers is not None:            # caller-mapped buffers (tests on one GPU: world 1)
            self._keep = buffers
            self.ptrs = [int(b.data_ptr()) for b in buffers]
            return
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        pg = group if group is not None else dist.group.WORLD
        handle = symm_mem.rendezvous(buf, pg.group_name)
        torch.cuda.synchronize(device)
        dist.barrier(group)                # every buffer is zero before any rank pushes
        self._keep = (buf, handle)
        self.ptrs = [int(x) for x in handle.buffer_ptrs]

    def decode(self, query, kv_cache_local, block_table_local, seq_lens_local, output, out_lse=None):
        """``query`` [batch, queries, heads, D] (the same on every rank); every rank gets ``output``."""
        from . import _cabi
        a = self.attn
        dev = query.device
        _cabi.decode_paged_exchange(query, a._as_bytes(kv_cache_local), block_table_local, seq_lens_local,
                                    a.signs(dev), a.scale, a.workspace(self.batch, dev, self.queries),
                                    self.rank, self.ptrs, self.nbytes, output, out_lse=out_lse,
                                    num_ctas=a.num_ctas, max_pages=block_table_local.shape[-1])
        return output

    def status(self) -> int:
        """Sticky status word of this rank's exchange buffer (0 ok, 1 a wait for a peer ran out)."""
        buf = self._keep[0]
        return int(buf[4:8].view(torch.int32).item())
