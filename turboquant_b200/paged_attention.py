"""Engine-independent core of the CUSTOM attention backend: cache layout, cache write and
paged decode over the 4-bit quantized KV cache, with workspaces cached per batch bucket.

This is the part of the reference's ``TurboQuantFusedImpl`` (turboquant/vllm_backend_fused.py:
93-468) that touches the quantized cache, without any vLLM type in its interface, so that the
benchmark and the tests can drive the same code the vLLM backend does.  All compute goes through
the C ABI (``_cabi``); there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import torch

from . import _cabi
from .synthetic import make_signs

TILE_DIMS = 64
QUANT_BYTES_PER_CHUNK = 32  # 64 dims x 4 bits / 8


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def slot_bytes(head_size: int) -> int:
    """Bytes per (token, head) cache slot: 32 code bytes + one fp16 norm per 64 dims, rounded up
    to 16 (vllm_backend_fused.py:64-72): 80 for head size 128."""
    dc = next_pow2(head_size) // TILE_DIMS
    raw = dc * QUANT_BYTES_PER_CHUNK + dc * 2
    return (raw + 15) & ~15


def kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int):
    return (2, num_blocks, block_size, num_kv_heads, slot_bytes(head_size))


class TurboQuantPagedAttention:
    """Cache write + decode attention for one attention layer geometry.

    ``write(key, value, kv_cache, slot_mapping)`` mirrors ``do_kv_cache_update`` and
    ``decode(query, kv_cache, block_table, seq_lens, output)`` the decode branch of ``forward``
    (vllm_backend_fused.py:308-322, 371-455).  Both launch on the current stream, allocate only on
    the first call of a batch bucket (before any graph capture, as the reference's ``_get_v5_ws``
    does) and never synchronise.
    """

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 seed: int = 42, num_ctas: int = 0):
        if not 32 < head_size <= 256:
            raise _cabi.TurboQuantError(f"head_size {head_size} is not supported (33..256; 128 and 96 run the tuned kernels)")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        self.padded_dim = next_pow2(head_size)
        self.seed = seed
        self.num_ctas = num_ctas
        self._signs: dict[torch.device, torch.Tensor] = {}
        self._workspaces: dict[tuple, torch.Tensor] = {}

    def signs(self, device) -> torch.Tensor:
        device = torch.device(device)
        s = self._signs.get(device)
        if s is None:
            s = make_signs(self.padded_dim, self.seed).to(device)
            self._signs[device] = s
        return s

    def workspace(self, batch: int, device, queries: int = 1) -> torch.Tensor:
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (device, batch, queries)
        ws = self._workspaces.get(key)
        if ws is None:
            nbytes = _cabi.decode_workspace_bytes(batch, queries * self.num_heads, self.num_kv_heads,
                                                  self.head_size, self.num_ctas)
            ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)  # zeroed once: the status word is sticky
            self._workspaces[key] = ws
        return ws

    @staticmethod
    def _as_bytes(kv_cache: torch.Tensor) -> torch.Tensor:
        return kv_cache if kv_cache.dtype == torch.uint8 else kv_cache.view(torch.uint8)

    def write(self, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
              slot_mapping: torch.Tensor, zero_pad: bool = False) -> None:
        n = slot_mapping.shape[0]
        if n == 0:
            return
        if key.dim() == 2:
            key = key.view(key.shape[0], self.num_kv_heads, self.head_size)
            value = value.view(value.shape[0], self.num_kv_heads, self.head_size)
        _cabi.write_kv_cache(self._as_bytes(kv_cache), key, value, self.signs(key.device), slot_mapping,
                             self.head_size, zero_pad=zero_pad)

    def decode(self, query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
               seq_lens: torch.Tensor, output: torch.Tensor | None = None,
               out_lse: torch.Tensor | None = None) -> torch.Tensor:
        if query.dim() == 4:
            return self.decode_shared(query, kv_cache, block_table, seq_lens, output, out_lse)
        if query.dim() == 2:
            query = query.view(query.shape[0], self.num_heads, self.head_size)
        if output is None:
            output = torch.empty_like(query)
        out3 = output.view(query.shape[0], self.num_heads, self.head_size)
        if block_table.dtype != torch.int32:
            block_table = block_table.to(torch.int32)
        if seq_lens.dtype != torch.int32:
            seq_lens = seq_lens.to(torch.int32)
        _cabi.decode_paged(query.contiguous(), self._as_bytes(kv_cache), block_table.contiguous(), seq_lens,
                           self.signs(query.device), self.scale, self.workspace(query.shape[0], query.device),
                           out3, out_lse=out_lse, num_ctas=self.num_ctas, max_pages=block_table.shape[-1])
        return output

    def decode_shared(self, query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
                      seq_lens: torch.Tensor, output: torch.Tensor | None = None,
                      out_lse: torch.Tensor | None = None) -> torch.Tensor:
        """Decode for ``query`` [batch, queries, heads, head_size] where the queries of one row share
        that row's KV (one ``seq_lens`` / ``block_table`` entry per row).  The reference would repeat
        the row ``queries`` times in the batch (its decode op has one query per batch row,
        csrc/src/decode_v5_tc_binding.cu:783-785) and stream the KV once per repeat; here the KV
        is streamed once.  queries x (heads / kv_heads) must not exceed 32 (8 for head sizes other than
        128 / 96 and for KV-head counts other than 2, 4, 8, 16: ``_cabi.decode_max_queries_per_seq``)."""
        B, NQ = query.shape[0], query.shape[1]
        if output is None:
            output = torch.empty_like(query)
        if block_table.dtype != torch.int32:
            block_table = block_table.to(torch.int32)
        if seq_lens.dtype != torch.int32:
            seq_lens = seq_lens.to(torch.int32)
        _cabi.decode_paged_multi(query.contiguous(), self._as_bytes(kv_cache), block_table.contiguous(), seq_lens,
                                 self.signs(query.device), self.scale, self.workspace(B, query.device, NQ),
                                 output.view(B, NQ, self.num_heads, self.head_size), out_lse=out_lse,
                                 num_ctas=self.num_ctas, max_pages=block_table.shape[-1])
        return output

    def decode_causal(self, query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
                      seq_lens: torch.Tensor, output: torch.Tensor | None = None,
                      out_lse: torch.Tensor | None = None) -> torch.Tensor:
        """Attention of the LAST ``queries`` tokens of every row's sequence over the quantized cache with
        a causal mask among them: ``query`` [batch, queries, heads, head_size]; the tokens' K / V are
        already in the cache and counted in ``seq_lens``.  One pass over the KV for
        queries x (heads / kv_heads) <= 32 query columns: a chunk of a continuing prefill, or the
        verification step of speculative decoding.  The reference's prefill ignores the cache
        (turboquant/vllm_backend_fused.py:336-369)."""
        B, NQ = query.shape[0], query.shape[1]
        if output is None:
            output = torch.empty_like(query)
        if block_table.dtype != torch.int32:
            block_table = block_table.to(torch.int32)
        if seq_lens.dtype != torch.int32:
            seq_lens = seq_lens.to(torch.int32)
        _cabi.decode_paged_causal(query.contiguous(), self._as_bytes(kv_cache), block_table.contiguous(), seq_lens,
                                  self.signs(query.device), self.scale, self.workspace(B, query.device, NQ),
                                  output.view(B, NQ, self.num_heads, self.head_size), out_lse=out_lse,
                                  num_ctas=self.num_ctas, max_pages=block_table.shape[-1])
        return output

    def dequant_cached(self, kv_cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                       cu_seqlens: torch.Tensor, total_tokens: int, dtype=torch.bfloat16):
        """Dense K / V ``[total_tokens, kv_heads, head_size]`` of the tokens already in the cache
        (row ``cu_seqlens[b] + t``), for a chunk of new queries that continues a prefill: concatenate
        with the chunk's fresh K / V and run a varlen attention kernel on the result.  The reference's
        prefill ignores the cache (vllm_backend_fused.py:336-369); this is the missing piece for
        chunked prefill over a quantized cache.  ``total_tokens`` is passed by the caller (no sync)."""
        dev = kv_cache.device
        k = torch.empty((total_tokens, self.num_kv_heads, self.head_size), dtype=dtype, device=dev)
        v = torch.empty_like(k)
        if total_tokens == 0:
            return k, v
        if block_table.dtype != torch.int32:
            block_table = block_table.to(torch.int32)
        _cabi.dequant_paged(self._as_bytes(kv_cache), block_table.contiguous(), seq_lens.to(torch.int32),
                            cu_seqlens.to(torch.int32), self.signs(dev), k, v, max_pages=block_table.shape[-1])
        return k, v

    def offload_pages(self, kv_cache: torch.Tensor, page_ids: torch.Tensor, host: torch.Tensor | None = None):
        """Packed copy of pages ``page_ids`` (K and V halves, 68 bytes per slot) in pinned host
        memory; asynchronous on the current stream (synchronise before reading ``host``).  The
        reference's offload study copies a whole slab, pad bytes included (tests/bench_kv_offload.py)."""
        _, _, bs, H, _ = kv_cache.shape
        n = page_ids.shape[0]
        nbytes = _cabi.pages_packed_bytes(n, bs, H, kv_cache.shape[-1]) if n else 0
        staging = torch.empty(nbytes, dtype=torch.uint8, device=kv_cache.device)
        if host is None:
            host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        if n:
            _cabi.pages_gather(self._as_bytes(kv_cache), page_ids.to(torch.int32), staging)
            host[:nbytes].copy_(staging, non_blocking=True)
        return host

    def restore_pages(self, kv_cache: torch.Tensor, page_ids: torch.Tensor, host: torch.Tensor) -> None:
        """Bring pages offloaded by ``offload_pages`` back into (possibly different) pages ``page_ids``."""
        _, _, bs, H, _ = kv_cache.shape
        n = page_ids.shape[0]
        if n == 0:
            return
        nbytes = _cabi.pages_packed_bytes(n, bs, H, kv_cache.shape[-1])
        staging = torch.empty(nbytes, dtype=torch.uint8, device=kv_cache.device)
        staging.copy_(host[:nbytes], non_blocking=True)
        _cabi.pages_scatter(self._as_bytes(kv_cache), page_ids.to(torch.int32), staging)

    def status(self, batch: int, device, queries: int = 1) -> int:
        """Status word the decode kernel leaves in its workspace (0 = ok); synchronises."""
        return int(self.workspace(batch, device, queries)[:4].view(torch.int32).item())
