"""CUSTOM vLLM attention backend over a single 4-bit quantized KV cache, with the class names,
methods and cache layout of the reference (turboquant/vllm_backend_fused.py:32-468).

    LLM(..., attention_backend="CUSTOM", kv_cache_dtype="fp8")

* ``TurboQuantBackend``: name "CUSTOM", cache shape ``(2, num_blocks, block_size, kv_heads, 80)`` and
  page size ``2 * block_size * kv_heads * 80`` bytes for the fp8 (1-byte) cache dtype.
* ``TurboQuantFusedImpl.do_kv_cache_update``: quantizes K and V of the step and scatters them into
  the cache (one launch; bf16/fp16 K/V and int64 slots are read as they are).
* ``TurboQuantFusedImpl.forward``: decode steps (``max_query_len == 1``) run the paged decode
  kernel on the quantized cache.  A prefill step whose sequences have nothing cached yet (known
  from the builder's host-side facts) runs FlashAttention on the step's fresh K/V, exactly as the
  reference does.  Any other step is a mixed step (``_mixed_step``): its decode rows go through the
  paged decode kernel, and every other row (first chunks, chunks that continue a sequence with
  cached context, which the reference does not handle: its prefill never reads the quantized
  cache, vllm_backend_fused.py:336-369) attends its cached tokens, dequantized into a dense varlen
  K/V (``tq_dequant_paged``), followed by the chunk's fresh K/V through the same varlen
  FlashAttention with bottom-right causal masking.
* ``TurboQuantMetadataBuilder``: the reference's is an empty subclass that sizes a uniform split
  count on the host; here the split plan is made inside the kernel from ``seq_lens``.  The builder
  adds what only the host knows without a synchronisation (``step_shape``): whether any sequence
  has cached context, how many rows are decode rows and how many dense K/V rows the others need.

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
    """Split planning needs nothing from the host (see the module docstring).  What the host does
    know at build time, and the kernels cannot tell the Python side without a synchronisation, is
    the shape of the step: whether any sequence has cached context, which rows are plain decode
    rows, and how many dense K/V rows the prefill rows need.  ``build`` attaches that as
    ``tq_step`` to the FlashAttention metadata; ``TurboQuantFusedImpl.forward`` works without it
    (it then takes the general path with a worst-case buffer)."""

    def build(self, common_prefix_len, common_attn_metadata, fast_build: bool = False):
        md = super().build(common_prefix_len, common_attn_metadata, fast_build)
        try:
            md.tq_step = step_shape(common_attn_metadata)
        except Exception:          # metadata without host copies: forward falls back to the general path
            pass
        return md


# Rows with cached context and at most this many new tokens (a short continuation chunk, the
# verification step of speculative decoding) attend over the quantized cache in one pass of the
# causal wide-tile decode kernel instead of a dequantized dense copy of their whole context.
FUSED_CHUNK_MAX = 8


def step_shape(common):
    """Host-side facts about a step from vLLM's CommonAttentionMetadata (its CPU copies of the query
    offsets and sequence lengths): a dict with ``any_cached`` (some sequence attends tokens that are
    only in the quantized cache), ``num_decode_rows`` (rows with one query token and cached context)
    ``num_short_rows`` (rows with 2 ... FUSED_CHUNK_MAX query tokens and cached context: they attend
    straight over the quantized cache with a causal mask among their tokens) and ``dense_rows`` (dense
    K/V rows the remaining rows need: the sum of their sequence lengths)."""
    qsl = common.query_start_loc_cpu
    n = int(common.num_reqs)
    q_lens = (qsl[1:n + 1] - qsl[:n]).to(torch.int64)
    seq = getattr(common, "seq_lens_cpu", None)
    if seq is None:
        seq = getattr(common, "_seq_lens_cpu", None)
    if seq is None:
        seq = common.seq_lens_cpu_upper_bound
    seq = seq[:n].to(torch.int64)
    cached = seq - q_lens
    is_decode = (q_lens == 1) & (cached > 0)
    is_short = (q_lens > 1) & (q_lens <= FUSED_CHUNK_MAX) & (cached > 0)
    dense = ~(is_decode | is_short)
    # an implementation without the causal kernel (``causal_chunk_supported``) treats the short rows as dense ones
    dense2 = ~is_decode
    return {"any_cached": bool((cached > 0).any()), "num_decode_rows": int(is_decode.sum()),
            "num_short_rows": int(is_short.sum()), "dense_rows": int(seq[dense].sum()),
            "max_prefill_seq": int(seq[dense].max()) if bool(dense.any()) else 0,
            "dense_rows_with_short": int(seq[dense2].sum()),
            "max_prefill_seq_with_short": int(seq[dense2].max()) if bool(dense2.any()) else 0}


def causal_chunk_supported(num_heads: int, num_kv_heads: int, head_size: int) -> bool:
    """Whether FUSED_CHUNK_MAX causal queries of a row fit one pass of the wide-tile decode kernel: head size
    128 or 96, 2 / 4 / 8 / 16 KV heads, and FUSED_CHUNK_MAX x (query heads per KV head) within its 32 columns."""
    from . import _cabi
    if head_size not in (128, 96) or num_kv_heads not in (2, 4, 8, 16):
        return False
    return _cabi.decode_max_queries_per_seq(num_heads, num_kv_heads) >= FUSED_CHUNK_MAX


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
        # short continuing chunks attend the quantized cache directly only where the causal kernel exists
        self._fuse_short = self._is_fp8 and causal_chunk_supported(self.num_heads, self.num_kv_heads, self.head_size)

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
            step = getattr(attn_metadata, "tq_step", None)
            if step is not None and not step["any_cached"]:
                # first chunks only: attention over the fresh K/V of this step, as the reference does
                # (vllm_backend_fused.py:336-369); the quantized cache is not read
                out = flash_attn_varlen_func(query[:n].view(n, self.num_heads, self.head_size),
                                             key[:n].view(n, self.num_kv_heads, self.head_size),
                                             value[:n].view(n, self.num_kv_heads, self.head_size),
                                             cu_seqlens_q=attn_metadata.query_start_loc,
                                             cu_seqlens_k=attn_metadata.query_start_loc,
                                             max_seqlen_q=attn_metadata.max_query_len,
                                             max_seqlen_k=attn_metadata.max_query_len,
                                             softmax_scale=self.scale, causal=True)
            else:
                # Some sequence may have cached context (known from the builder, or not known at all:
                # the two maxima of the metadata cannot rule it out, a long first chunk hides a short
                # continuation): decode rows go through the paged decode kernel, every other row
                # attends its dequantized cached tokens followed by the chunk's fresh K/V.
                out = self._mixed_step(query[:n], key[:n], value[:n], kv_cache, attn_metadata, step,
                                       flash_attn_varlen_func)
            output[:n] = out.to(output.dtype).view(output[:n].shape)
            return output
        q = query[:n].view(n, self.num_heads, self.head_size)
        if output is None:
            output = torch.empty_like(query[:n])
        out = output[:n].view(n, self.num_heads, self.head_size)
        self._attn.decode(q, kv_cache, attn_metadata.block_table[:n], attn_metadata.seq_lens[:n], out)
        return output

    def _mixed_step(self, query, key, value, kv_cache, md, step, flash_attn_varlen_func):
        """A step whose sequences may have cached context: prefill chunks, continuing chunks and
        decode rows in any mix.  No host synchronisation; every shape comes from the metadata.

        * Decode rows (one query token, cached context) run through the paged decode kernel over
          the quantized cache: all rows are handed to it with the length of every other row set
          to zero, and their outputs are dropped.
        * Rows with cached context and 2 ... FUSED_CHUNK_MAX new tokens run through the causal
          wide-tile decode kernel: their tokens are already in the cache, the row's queries are
          padded at the front to FUSED_CHUNK_MAX (a pad query sees fewer tokens than the first real
          one and its output is dropped), every other row has length zero there.  Geometries without that
          kernel (``causal_chunk_supported``: other head sizes, more than four query heads per KV head, KV
          head counts the wide tile does not take) send these rows the dense way below.
        * Every other row b contributes ``seq_lens[b]`` keys to a dense varlen K/V: its cached
          tokens, dequantized from the cache, then the chunk's own fresh K/V (the chunk is already
          in the cache as well, quantized; its fresh values are used, as a first chunk would).  The
          buffer has ``step["dense_rows"]`` rows when the builder attached the step's shape, else
          the ``batch x max_seq_len`` bound (rows beyond ``cu_k[-1]`` are unused)."""
        dev = query.device
        n = query.shape[0]
        qsl = md.query_start_loc.to(torch.int32)
        B = qsl.shape[0] - 1
        seq_lens = md.seq_lens[:B].to(torch.int32)
        q_lens = qsl[1:] - qsl[:-1]
        cached = seq_lens - q_lens
        is_dec = (q_lens == 1) & (cached > 0)
        is_short = (q_lens > 1) & (q_lens <= FUSED_CHUNK_MAX) & (cached > 0)
        if not self._fuse_short:      # no causal kernel for this geometry: those rows go the dense way
            is_short = torch.zeros_like(is_short)
        fused = is_dec | is_short
        zero = torch.zeros_like(seq_lens)
        bt = md.block_table[:B]
        if bt.dtype != torch.int32:
            bt = bt.to(torch.int32)
        bt = bt.contiguous()
        q3 = query.view(n, self.num_heads, self.head_size)
        first_tok = qsl[:-1].long()

        # ---- prefill / continuation rows: dense K/V = dequantized cached tokens + fresh chunk -------
        pf_seq = torch.where(fused, zero, seq_lens)
        pf_cached = torch.where(fused, zero, cached)
        cu_k = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        cu_k[1:] = torch.cumsum(pf_seq, 0)
        max_seq_len = int(getattr(md, "max_seq_len", md.max_query_len))
        if step is not None and self._fuse_short:
            rows, max_k = max(step["dense_rows"], 1), max(step["max_prefill_seq"], 1)
        elif step is not None and "dense_rows_with_short" in step:
            rows, max_k = max(step["dense_rows_with_short"], 1), max(step["max_prefill_seq_with_short"], 1)
        else:
            rows, max_k = B * max_seq_len, max_seq_len
        # one spare row at the end takes the fresh K/V of the decode and short rows' tokens, which nobody reads
        k_all = torch.empty((rows + 1, self.num_kv_heads, self.head_size), dtype=query.dtype, device=dev)
        v_all = torch.empty_like(k_all)
        from . import _cabi
        _cabi.dequant_paged(self._attn._as_bytes(kv_cache), bt, pf_cached.contiguous(), cu_k,
                            self._attn.signs(dev), k_all, v_all, max_pages=bt.shape[-1])
        # the chunk's fresh rows go behind the cached rows of their sequence
        tok = torch.arange(n, device=dev, dtype=torch.int32)
        seq_of = torch.bucketize(tok, qsl[1:], right=True)
        dest = (cu_k[:-1][seq_of] + pf_cached[seq_of] + (tok - qsl[:-1][seq_of])).long()
        dest = torch.where(fused[seq_of], torch.full_like(dest, rows), dest)
        k_all[dest] = key.view(n, self.num_kv_heads, self.head_size).to(k_all.dtype)
        v_all[dest] = value.view(n, self.num_kv_heads, self.head_size).to(v_all.dtype)
        out = flash_attn_varlen_func(q3, k_all, v_all, cu_seqlens_q=qsl, cu_seqlens_k=cu_k,
                                     max_seqlen_q=md.max_query_len, max_seqlen_k=max_k,
                                     softmax_scale=self.scale, causal=True)
        # ---- decode rows: the paged decode kernel, one query per row, other rows masked out ---------
        if step is None or step["num_decode_rows"] > 0:
            dec_lens = torch.where(is_dec, seq_lens, zero).contiguous()
            q_rows = q3[first_tok].contiguous()
            dec_out = torch.empty_like(q_rows)
            self._attn.decode(q_rows, kv_cache, bt, dec_lens, dec_out)
            out[first_tok] = torch.where(is_dec[:, None, None], dec_out.to(out.dtype), out[first_tok])
        # ---- short rows: causal queries over the quantized cache, padded at the front --------------
        if self._fuse_short and (step is None or step.get("num_short_rows", 0) > 0):
            nq = FUSED_CHUNK_MAX
            slot = (seq_of * nq + (nq - q_lens[seq_of]) + (tok - qsl[:-1][seq_of])).long()
            slot = torch.where(is_short[seq_of], slot, torch.full_like(slot, B * nq))   # others: the spare row
            q_pad = torch.zeros((B * nq + 1, self.num_heads, self.head_size), dtype=query.dtype, device=dev)
            q_pad[slot] = q3
            short_lens = torch.where(is_short, seq_lens, zero).contiguous()
            short_out = torch.empty((B, nq, self.num_heads, self.head_size), dtype=query.dtype, device=dev)
            self._attn.decode_causal(q_pad[:B * nq].view(B, nq, self.num_heads, self.head_size), kv_cache, bt,
                                     short_lens, short_out)
            picked = short_out.view(B * nq, self.num_heads, self.head_size)[slot.clamp(max=B * nq - 1)]
            out = torch.where(is_short[seq_of][:, None, None], picked.to(out.dtype), out)
        return out
