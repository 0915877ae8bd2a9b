"""CUSTOM vLLM attention backend over a single 4-bit quantized KV cache, with the class names,
methods and cache layout of the reference (turboquant/vllm_backend_fused.py:32-468).

    LLM(..., attention_backend="CUSTOM", kv_cache_dtype="fp8")

* ``TurboQuantBackend``: name "CUSTOM", cache shape ``(2, num_blocks, block_size, kv_heads, 80)`` and
  page size ``2 * block_size * kv_heads * 80`` bytes for the fp8 (1-byte) cache dtype.
* ``TurboQuantFusedImpl.do_kv_cache_update``: quantizes K and V of the step and scatters them into
  the cache (one launch; bf16/fp16 K/V and int64 slots are read as they are).
* ``TurboQuantFusedImpl.forward``: decode steps (``max_query_len == 1``) run the paged decode
  kernel on the quantized cache.  A prefill step whose sequences have nothing cached yet runs
  FlashAttention on the step's fresh K/V, exactly as the reference does.  A prefill chunk that
  continues sequences with cached context (which the reference does not handle: its prefill never
  reads the quantized cache, vllm_backend_fused.py:336-369) first dequantizes the cached tokens
  into a dense varlen K/V (``tq_dequant_paged``), puts the chunk's fresh K/V behind them and runs
  the same varlen FlashAttention with bottom-right causal masking.
* ``TurboQuantMetadataBuilder``: the reference's is an empty subclass that sizes a uniform split
  count on the host; here the split plan is made inside the kernel from ``seq_lens``, so the
  builder only has to keep the FlashAttention metadata (block table, lengths) as it is.

All cache work goes through ``TurboQuantPagedAttention`` (C ABI); a failure raises, there is no
fallback to another backend for a quantized cache.
"""
from __future__ import annotations

import torch
from vllm.v1.attention.backends.flash_attn import (FlashAttentionBackend, FlashAttentionImpl,
                                                   FlashAttentionMetadataBuilder)

from .paged_attention import TurboQuantPagedAttention, next_pow2, slot_bytes

TILE_DIMS = 64
QUANT_BYTES_PER_CHUNK = 32
_FP8 = ("fp8", "fp8_e4m3")


def _next_pow2(n):
    return next_pow2(n)


class TurboQuantBackend(FlashAttentionBackend):
    # vLLM calls do_kv_cache_update separately from forward
    forward_includes_kv_cache_update = False

    @staticmethod
    def get_name():
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return TurboQuantFusedImpl

    @staticmethod
    def get_builder_cls():
        return TurboQuantMetadataBuilder

    @classmethod
    def supports_kv_cache_dtype(cls, kv_cache_dtype) -> bool:
        if kv_cache_dtype in _FP8:
            return True
        return super().supports_kv_cache_dtype(kv_cache_dtype)

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if cache_dtype_str in _FP8:
            return (2, num_blocks, block_size, num_kv_heads, slot_bytes(head_size))
        return FlashAttentionBackend.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size,
                                                        cache_dtype_str)

    @classmethod
    def get_kv_cache_page_size(cls, block_size, num_kv_heads, head_size, dtype, cache_dtype_str="auto"):
        if cache_dtype_str in _FP8:
            return 2 * block_size * num_kv_heads * slot_bytes(head_size)
        return None


class TurboQuantMetadataBuilder(FlashAttentionMetadataBuilder):
    """Split planning needs nothing from the host (see the module docstring)."""


class TurboQuantFusedImpl(FlashAttentionImpl):
    def __init__(self, num_heads, head_size, scale, num_kv_heads, alibi_slopes, sliding_window,
                 kv_cache_dtype, *args, **kwargs):
        self._real_cache_dtype = kv_cache_dtype
        self._is_fp8 = kv_cache_dtype in _FP8
        parent_dtype = "auto" if self._is_fp8 else kv_cache_dtype   # the parent must not see fp8
        super().__init__(num_heads, head_size, scale, num_kv_heads, alibi_slopes, sliding_window,
                         parent_dtype, *args, **kwargs)
        self.kv_cache_dtype = self._real_cache_dtype
        self._pd = _next_pow2(self.head_size)
        self._dc = self._pd // TILE_DIMS
        self._qbytes = self._dc * QUANT_BYTES_PER_CHUNK
        self._nbytes = self._dc * 2
        self._attn = (TurboQuantPagedAttention(self.num_heads, self.head_size, self.scale, self.num_kv_heads)
                      if self._is_fp8 else None)

    @staticmethod
    def _choose_num_splits(batch_size: int, max_len: int, num_kv_heads: int, device) -> int:
        """Kept for interface compatibility: the kernel balances page ranges over one thread
        block per SM by itself, so the number of pieces per sequence is ``SMs / batch`` on average."""
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        return max(1, min(sms // max(batch_size, 1), max(1, max_len // 128)))

    @torch.no_grad()
    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        if not self._is_fp8:
            return super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
        n = slot_mapping.shape[0]
        self._attn.write(key[:n], value[:n], kv_cache, slot_mapping)

    @torch.no_grad()
    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None, **kwargs):
        if attn_metadata is None:
            return torch.zeros_like(query) if output is None else output
        if not self._is_fp8:
            return super().forward(layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                                   output_block_scale, **kwargs)
        n = attn_metadata.num_actual_tokens
        if attn_metadata.max_query_len != 1:
            from vllm.vllm_flash_attn import flash_attn_varlen_func
            if output is None:
                output = torch.empty_like(query[:n])
            max_seq_len = getattr(attn_metadata, "max_seq_len", attn_metadata.max_query_len)
            if max_seq_len > attn_metadata.max_query_len:
                out = self._continuation_prefill(query[:n], key[:n], value[:n], kv_cache, attn_metadata, max_seq_len,
                                                 flash_attn_varlen_func)
                output[:n] = out.to(output.dtype).view(output[:n].shape)
                return output
            # first chunk: attention over the fresh K/V of this step; the quantized cache is not read
            out = flash_attn_varlen_func(query[:n], key[:n], value[:n],
                                         cu_seqlens_q=attn_metadata.query_start_loc,
                                         cu_seqlens_k=attn_metadata.query_start_loc,
                                         max_seqlen_q=attn_metadata.max_query_len,
                                         max_seqlen_k=attn_metadata.max_query_len,
                                         softmax_scale=self.scale, causal=True)
            output[:n] = out.to(output.dtype).view(output[:n].shape)
            return output
        q = query[:n].view(n, self.num_heads, self.head_size)
        if output is None:
            output = torch.empty_like(query[:n])
        out = output[:n].view(n, self.num_heads, self.head_size)
        self._attn.decode(q, kv_cache, attn_metadata.block_table[:n], attn_metadata.seq_lens[:n], out)
        return output

    def _continuation_prefill(self, query, key, value, kv_cache, md, max_seq_len, flash_attn_varlen_func):
        """Chunk of new tokens over sequences with cached context.  Sequence b contributes
        ``seq_lens[b]`` keys: its ``seq_lens[b] - q_len[b]`` cached tokens, dequantized from the
        cache, then the chunk's own fresh K/V (the chunk is already in the cache as well, quantized;
        its fresh values are used, as a first chunk would).  No host synchronisation: the dense
        buffer is sized by the ``batch x max_seq_len`` bound, rows beyond ``cu_k[-1]`` are unused."""
        dev = query.device
        qsl = md.query_start_loc.to(torch.int32)
        B = qsl.shape[0] - 1
        seq_lens = md.seq_lens[:B].to(torch.int32)
        q_lens = qsl[1:] - qsl[:-1]
        cached = seq_lens - q_lens
        cu_k = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        cu_k[1:] = torch.cumsum(seq_lens, 0)
        rows = B * int(max_seq_len)
        k_all = torch.empty((rows, self.num_kv_heads, self.head_size), dtype=query.dtype, device=dev)
        v_all = torch.empty_like(k_all)
        from . import _cabi
        bt = md.block_table[:B]
        if bt.dtype != torch.int32:
            bt = bt.to(torch.int32)
        _cabi.dequant_paged(self._attn._as_bytes(kv_cache), bt.contiguous(), cached.contiguous(), cu_k,
                            self._attn.signs(dev), k_all, v_all, max_pages=bt.shape[-1])
        # fresh rows of the chunk go behind the cached rows of their sequence
        n = query.shape[0]
        tok = torch.arange(n, device=dev, dtype=torch.int32)
        seq_of = torch.bucketize(tok, qsl[1:], right=True)
        dest = (cu_k[:-1][seq_of] + cached[seq_of] + (tok - qsl[:-1][seq_of])).long()
        k_all[dest] = key.view(n, self.num_kv_heads, self.head_size).to(k_all.dtype)
        v_all[dest] = value.view(n, self.num_kv_heads, self.head_size).to(v_all.dtype)
        return flash_attn_varlen_func(query.view(n, self.num_heads, self.head_size), k_all, v_all,
                                      cu_seqlens_q=qsl, cu_seqlens_k=cu_k, max_seqlen_q=md.max_query_len,
                                      max_seqlen_k=int(max_seq_len), softmax_scale=self.scale, causal=True)
