"""ctypes binding of libturboquant_b200.so (the C ABI declared in include/turboquant_b200.h).

torch is used for device memory and the current stream only: every call passes raw device
pointers, sizes and the stream handle.  There is no CPU fallback: if the library is missing or
a tensor is not on a CUDA device the call raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

import os

_PKG = Path(__file__).resolve().parent
# TURBOQUANT_B200_LIB points at another build of the same library (e.g. an experimental variant)
LIB_PATH = Path(os.environ.get("TURBOQUANT_B200_LIB", _PKG / "lib" / "libturboquant_b200.so"))

TQ_F32, TQ_F16, TQ_BF16 = 0, 1, 2
TQ_I32, TQ_I64 = 0, 1
TQ_PACK_LOW_FIRST, TQ_PACK_CACHE = 0, 1
TQ_WRITE_ZERO_PAD, TQ_WRITE_EXACT_PATH, TQ_WRITE_TENSOR_PATH = 1, 2, 4
STATIC_SCRATCH_BYTES = 8 << 20  # TQ_STATIC_SCRATCH_BYTES

_DTYPES = {torch.float32: TQ_F32, torch.float16: TQ_F16, torch.bfloat16: TQ_BF16}

EXPORTS = (
    "tq_abi_version", "tq_last_error", "tq_codebook", "tq_write_kv_cache", "tq_quantize_flat",
    "tq_dequantize_flat", "tq_fwht", "tq_decode_workspace_bytes", "tq_decode_paged",
    "tq_decode_paged_partial", "tq_merge_rotated", "tq_debug_set_decode_events",
    "tq_decode_paged_static", "tq_decode_paged_multi", "tq_decode_paged_causal", "tq_nc_slot_bytes",
    "tq_nc_write_kv_cache", "tq_nc_decode_workspace_bytes", "tq_nc_decode_paged", "tq_nc_write_dropped", "tq_exchange_bytes", "tq_decode_paged_exchange",
    "tq_dequant_paged", "tq_pages_packed_bytes", "tq_pages_gather", "tq_pages_scatter",
    "tq_decode_max_query_columns", "tq_set_exchange_wait_limit", "tq_decode_static_status", "tq_fault_counts",
    "tq_write_guard_stats", "tq_pages_packed_bytes_for_slot",
)

_lib = None


class TurboQuantError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load the library or fail loudly (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise TurboQuantError(
                f"{LIB_PATH} is missing: build it with `python -m turboquant_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(str(LIB_PATH))
        L.tq_last_error.restype = ctypes.c_char_p
        L.tq_decode_workspace_bytes.restype = ctypes.c_size_t
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise TurboQuantError(f"turboquant_b200 error {rc}: {lib().tq_last_error().decode()}")


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _cuda(t: torch.Tensor, name: str) -> None:
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise TurboQuantError(f"{name} must be a CUDA tensor (no CPU fallback)")


def debug_checks() -> bool:
    """TQ_DEBUG_CHECKS=1 makes every call validate its index tensors on the host first (minimum /
    maximum of slots, page ids and lengths against the cache geometry).  Each check synchronises,
    so this is for bringing up an integration, not for serving; inside a stream capture, where a
    synchronisation is illegal, the checks are skipped."""
    if os.environ.get("TQ_DEBUG_CHECKS", "0") in ("", "0"):
        return False
    return not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())


def _check_slots(slot_mapping: torch.Tensor, num_blocks: int, block_size: int) -> None:
    if slot_mapping.numel() and int(slot_mapping.max().item()) >= num_blocks * block_size:
        raise TurboQuantError(f"slot_mapping holds slot {int(slot_mapping.max().item())} but the cache has "
                              f"{num_blocks} x {block_size} = {num_blocks * block_size} slots")


def _check_pages(page_indices, page_indptr, max_pages, seq_lens, num_blocks: int, block_size: int) -> None:
    lens = seq_lens.to(torch.int64)
    if lens.numel() and int(lens.min().item()) < 0:
        raise TurboQuantError("seq_lens holds a negative length")
    need = (lens + block_size - 1) // block_size
    if page_indptr is None:
        if lens.numel() and int(need.max().item()) > max_pages:
            raise TurboQuantError(f"a sequence needs {int(need.max().item())} pages but the block table has {max_pages} per row")
        rows = page_indices.reshape(lens.numel(), -1)[:, :max_pages].to(torch.int64)
        used = torch.arange(rows.shape[1], device=rows.device)[None, :] < need[:, None]
        ids = rows[used]
    else:
        ptr = page_indptr.to(torch.int64)
        have = ptr[1:] - ptr[:-1]
        if bool((need > have[: need.numel()]).any().item()):
            raise TurboQuantError("a sequence is longer than its page list (page_indptr)")
        ids = page_indices[: int(ptr[-1].item())].to(torch.int64)
    if ids.numel() and (int(ids.min().item()) < 0 or int(ids.max().item()) >= num_blocks):
        raise TurboQuantError(f"page id out of range: [{int(ids.min().item())}, {int(ids.max().item())}] "
                              f"with {num_blocks} pages in the cache")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TurboQuantError(f"unsupported dtype {dt}") from None


def codebook(dim: int, bits: int):
    """(centroids, boundaries) as CPU fp32 tensors; host-side call."""
    cen = (ctypes.c_float * (1 << bits))()
    bnd = (ctypes.c_float * ((1 << bits) - 1))()
    _check(lib().tq_codebook(ctypes.c_int(dim), ctypes.c_int(bits), cen, bnd))
    return torch.tensor(list(cen), dtype=torch.float32), torch.tensor(list(bnd), dtype=torch.float32)


def write_kv_cache(kv_cache: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                   signs: torch.Tensor, slot_mapping: torch.Tensor, head_dim: int,
                   zero_pad: bool = False, path: str = "auto") -> None:
    """kv_cache uint8-addressable [2, nb, bs, H, slot]; key/value [T, H, D] (token stride free).
    ``path``: "auto" (large fp16 / bf16 writes take the tensor-core kernel), "exact" or "tensor";
    all three produce the same bytes."""
    for t, n in ((kv_cache, "kv_cache"), (key, "key"), (value, "value"), (signs, "signs"),
                 (slot_mapping, "slot_mapping")):
        _cuda(t, n)
    if kv_cache.dim() != 5 or kv_cache.shape[0] != 2 or not kv_cache.is_contiguous():
        raise TurboQuantError("kv_cache must be a contiguous [2, num_blocks, block_size, heads, slot_bytes] tensor")
    if kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must have a 1-byte element type")
    _, nb, bs, H, ebs = kv_cache.shape
    T = slot_mapping.shape[0]
    if key.dtype != value.dtype:
        raise TurboQuantError("key and value must share a dtype")
    for t, n in ((key, "key"), (value, "value")):
        if t.dim() != 3 or t.shape[1] != H or t.shape[2] != head_dim or t.shape[0] < T:
            raise TurboQuantError(f"{n} must be [>=num_tokens, {H}, {head_dim}], got {tuple(t.shape)}")
        if t.stride(2) != 1 or t.stride(1) != head_dim:
            raise TurboQuantError(f"{n}: heads of one token must be contiguous")
    padded = 1 << (head_dim - 1).bit_length()
    if signs.dtype != torch.float32 or signs.numel() < padded or not signs.is_contiguous():
        raise TurboQuantError(f"signs must be contiguous fp32 with {padded} entries (the padded head size)")
    if slot_mapping.dtype not in (torch.int32, torch.int64) or not slot_mapping.is_contiguous():
        raise TurboQuantError("slot_mapping must be contiguous int32 or int64")
    if debug_checks():
        _check_slots(slot_mapping, nb, bs)
    _check(lib().tq_write_kv_cache(
        _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(H), ctypes.c_int(ebs),
        _ptr(key), _ptr(value), ctypes.c_int(dtype_code(key.dtype)), ctypes.c_int64(T),
        ctypes.c_int64(key.stride(0)), ctypes.c_int64(value.stride(0)), _ptr(signs),
        _ptr(slot_mapping), ctypes.c_int(TQ_I64 if slot_mapping.dtype == torch.int64 else TQ_I32),
        ctypes.c_int(head_dim),
        ctypes.c_int((TQ_WRITE_ZERO_PAD if zero_pad else 0) | {"auto": 0, "exact": TQ_WRITE_EXACT_PATH,
                                                                "tensor": TQ_WRITE_TENSOR_PATH}[path]),
        _stream(kv_cache)))


def quantize_flat(x: torch.Tensor, signs: torch.Tensor, bits: int, cache_order: bool = False):
    _cuda(x, "x")
    _cuda(signs, "signs")
    x = x.contiguous()
    dim = x.shape[-1]
    padded = 1 if dim <= 1 else 1 << (dim - 1).bit_length()
    n = x.numel() // dim if dim else 0
    vpb = 8 // bits
    nbytes = (padded + vpb - 1) // vpb
    packed = torch.empty(x.shape[:-1] + (nbytes,), dtype=torch.uint8, device=x.device)
    norms = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _check(lib().tq_quantize_flat(
        _ptr(x), ctypes.c_int(dtype_code(x.dtype)), ctypes.c_int64(n), ctypes.c_int(dim), _ptr(signs),
        ctypes.c_int(bits), ctypes.c_int(TQ_PACK_CACHE if cache_order else TQ_PACK_LOW_FIRST),
        _ptr(packed), _ptr(norms), _stream(x)))
    return packed, norms


def dequantize_flat(packed: torch.Tensor, norms: torch.Tensor, signs: torch.Tensor, dim: int,
                    bits: int, cache_order: bool = False) -> torch.Tensor:
    _cuda(packed, "packed")
    _cuda(norms, "norms")
    packed = packed.contiguous()
    norms = norms.to(torch.float32).contiguous()
    n = norms.numel()
    out = torch.empty(norms.shape + (dim,), dtype=torch.float32, device=packed.device)
    _check(lib().tq_dequantize_flat(
        _ptr(packed), _ptr(norms), ctypes.c_int64(n), ctypes.c_int(dim), _ptr(signs),
        ctypes.c_int(bits), ctypes.c_int(TQ_PACK_CACHE if cache_order else TQ_PACK_LOW_FIRST),
        _ptr(out), _stream(packed)))
    return out


def fwht(x: torch.Tensor, padded_dim: int, out_dim: int, pre_signs=None, post_signs=None) -> torch.Tensor:
    _cuda(x, "x")
    xf = x.to(torch.float32).contiguous()
    in_dim = xf.shape[-1]
    n = xf.numel() // in_dim if in_dim else 0
    out = torch.empty(xf.shape[:-1] + (out_dim,), dtype=torch.float32, device=x.device)
    _check(lib().tq_fwht(_ptr(xf), ctypes.c_int64(n), ctypes.c_int(in_dim), ctypes.c_int(padded_dim),
                         ctypes.c_int(out_dim), _ptr(pre_signs), _ptr(post_signs), _ptr(out), _stream(x)))
    return out


def decode_workspace_bytes(batch: int, num_q_heads: int, num_kv_heads: int, head_dim: int = 128,
                           num_ctas: int = 0) -> int:
    return int(lib().tq_decode_workspace_bytes(ctypes.c_int(batch), ctypes.c_int(num_q_heads),
                                               ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
                                               ctypes.c_int(num_ctas)))


def _decode_args(q, kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs):
    for t, n in ((q, "q"), (kv_cache, "kv_cache"), (page_indices, "page_indices"),
                 (seq_lens, "seq_lens"), (signs, "signs")):
        _cuda(t, n)
    if q.dim() != 3 or not q.is_contiguous():
        raise TurboQuantError("q must be contiguous [batch, num_q_heads, head_dim]")
    if kv_cache.dim() != 5 or kv_cache.shape[0] != 2 or not kv_cache.is_contiguous() or kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must be contiguous 1-byte [2, num_blocks, block_size, heads, slot_bytes]")
    if page_indices.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TurboQuantError("page_indices and seq_lens must be int32")
    if not page_indices.is_contiguous() or not seq_lens.is_contiguous():
        raise TurboQuantError("page_indices and seq_lens must be contiguous")
    if page_indptr is not None and (page_indptr.dtype != torch.int32 or not page_indptr.is_cuda):
        raise TurboQuantError("page_indptr must be a CUDA int32 tensor")
    if seq_lens.shape[0] != q.shape[0]:
        raise TurboQuantError("seq_lens must have one entry per query row")
    if debug_checks():
        _check_pages(page_indices, page_indptr, max_pages, seq_lens, kv_cache.shape[1], kv_cache.shape[2])


def decode_max_queries_per_seq(num_q_heads: int, num_kv_heads: int, head_size: int = 128) -> int:
    """How many decode queries that share one sequence's KV fit one pass of ``decode_paged_multi``:
    the wide-tile kernel (up to ``tq_decode_max_query_columns()`` columns) takes 2, 4, 8 or 16 KV heads at head
    size 128 / 96; any other KV-head count or head size keeps the 8 columns of the mma.sync kernels."""
    wide = num_kv_heads in (2, 4, 8, 16) and head_size in (128, 96)
    cols = int(lib().tq_decode_max_query_columns()) if wide else 8
    return max(1, cols // max(1, num_q_heads // num_kv_heads))


def fault_counts():
    """(dropped cache-write tokens, skipped dequant page halves, skipped offload pages) that the
    kernels caught as out-of-range indices since the library was loaded; synchronises."""
    c = (ctypes.c_int32 * 3)()
    _check(lib().tq_fault_counts(c))
    return tuple(int(x) for x in c)


def write_guard_stats():
    """(rows the tensor-core write kernel processed, rows it re-derived exactly); synchronises."""
    a, b = ctypes.c_int64(0), ctypes.c_int64(0)
    _check(lib().tq_write_guard_stats(ctypes.byref(a), ctypes.byref(b)))
    return int(a.value), int(b.value)


def set_exchange_wait_limit(polls: int) -> None:
    """Polls (256 ns apart) the KV-split exchange may wait for a peer's partial; 0 = default."""
    _check(lib().tq_set_exchange_wait_limit(ctypes.c_int(polls)))


def decode_paged(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, workspace, out,
                 page_indptr=None, max_pages: int | None = None, out_lse=None, num_ctas: int = 0):
    """One decode step; writes ``out`` [batch, Hq, D] (and ``out_lse`` fp32 [batch, Hq])."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    _decode_args(q, kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    _check(lib().tq_decode_paged(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(H),
        ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens), _ptr(signs),
        ctypes.c_float(sm_scale), _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        _ptr(out), ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse), ctypes.c_int(num_ctas), _stream(q)))
    return out


def _check_rotated_partial(out_rot, head_dim: int):
    """A rotated-domain partial is as wide as the padded head: 128 for head sizes 65 ... 128, else 64 or 256."""
    padded = 64 if head_dim <= 64 else 128 if head_dim <= 128 else 256
    if out_rot.dtype != torch.float32 or out_rot.shape[-1] != padded or not out_rot.is_contiguous():
        raise TurboQuantError(f"a rotated partial must be contiguous fp32 with a last dim of {padded} "
                              f"(the padded head size), got {tuple(out_rot.shape)} {out_rot.dtype}")


def decode_paged_multi(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, workspace, out,
                       page_indptr=None, max_pages: int | None = None, out_lse=None, num_ctas: int = 0,
                       kv_begin: int = 0, kv_end: int = -1, rotated_partial: bool = False):
    """One decode step for sequences that carry several queries sharing their KV: ``q`` and ``out``
    are [batch, queries, Hq, D], ``out_lse`` fp32 [batch, queries, Hq]; queries x (Hq / H) <= 32 (more than 8: the wide-tile kernel).
    The workspace is sized for queries x Hq heads.  ``rotated_partial``: fp32 rotated-domain
    partial + base-2 LSE over tokens [kv_begin, kv_end), as ``decode_paged_partial``."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    if q.dim() != 4:
        raise TurboQuantError("q must be [batch, queries, num_q_heads, head_dim]")
    if not q.is_contiguous():
        raise TurboQuantError("q must be contiguous")
    _decode_args(q.view(q.shape[0], -1, q.shape[3]), kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, NQ, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    if rotated_partial:
        _check_rotated_partial(out, D)
    _check(lib().tq_decode_paged_multi(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(NQ), ctypes.c_int(Hq),
        ctypes.c_int(H), ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens),
        ctypes.c_int64(kv_begin), ctypes.c_int64(kv_end), _ptr(signs),
        ctypes.c_float(sm_scale), _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        _ptr(out), ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse), ctypes.c_int(1 if rotated_partial else 0),
        ctypes.c_int(num_ctas), _stream(q)))
    return out


def decode_paged_causal(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, workspace, out,
                        page_indptr=None, max_pages: int | None = None, out_lse=None, num_ctas: int = 0):
    """``decode_paged_multi`` with a causal mask among the queries of a row: ``q`` [batch, queries, Hq, D]
    holds the last ``queries`` tokens of every sequence (already written to the cache and counted in
    ``seq_lens``); query i sees the first ``seq_len - (queries - 1 - i)`` tokens."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    if q.dim() != 4:
        raise TurboQuantError("q must be [batch, queries, num_q_heads, head_dim]")
    if not q.is_contiguous():
        raise TurboQuantError("q must be contiguous")
    _decode_args(q.view(q.shape[0], -1, q.shape[3]), kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, NQ, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    _check(lib().tq_decode_paged_causal(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(NQ), ctypes.c_int(Hq),
        ctypes.c_int(H), ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens), _ptr(signs),
        ctypes.c_float(sm_scale), _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        _ptr(out), ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse), ctypes.c_int(num_ctas), _stream(q)))
    return out


def dequant_paged(kv_cache, page_indices, seq_lens, cu_seqlens, signs, k_out, v_out, page_indptr=None,
                  max_pages: int | None = None):
    """Cached tokens of every sequence -> dense K / V ``[total_tokens, H, 128]`` (row
    ``cu_seqlens[b] + t``), dequantized; ``k_out`` / ``v_out`` fp32, fp16 or bf16, last two dims
    contiguous."""
    for t, n in ((kv_cache, "kv_cache"), (page_indices, "page_indices"), (seq_lens, "seq_lens"),
                 (cu_seqlens, "cu_seqlens"), (signs, "signs"), (k_out, "k_out"), (v_out, "v_out")):
        _cuda(t, n)
    if kv_cache.dim() != 5 or kv_cache.shape[0] != 2 or not kv_cache.is_contiguous() or kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must be contiguous 1-byte [2, num_blocks, block_size, heads, slot_bytes]")
    for t, n in ((page_indices, "page_indices"), (seq_lens, "seq_lens"), (cu_seqlens, "cu_seqlens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise TurboQuantError(f"{n} must be contiguous int32")
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    _, nb, bs, H, ebs = kv_cache.shape
    B = seq_lens.shape[0]
    if cu_seqlens.shape[0] != B + 1:
        raise TurboQuantError("cu_seqlens must have batch + 1 entries")
    if k_out.dim() != 3 or k_out.shape != v_out.shape or k_out.dtype != v_out.dtype or k_out.shape[1] != H \
            or k_out.stride(2) != 1 or k_out.stride(1) != k_out.shape[2] or v_out.stride() != k_out.stride():
        raise TurboQuantError("k_out / v_out must be [tokens, H, D] with contiguous heads and equal layout")
    _check(lib().tq_dequant_paged(
        _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(H), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens), _ptr(cu_seqlens),
        ctypes.c_int(B), _ptr(signs), ctypes.c_int(k_out.shape[2]), _ptr(k_out), _ptr(v_out),
        ctypes.c_int(dtype_code(k_out.dtype)), ctypes.c_int64(k_out.stride(0)), _stream(kv_cache)))
    return k_out, v_out


def pages_packed_bytes(n_pages: int, block_size: int, num_kv_heads: int, slot_bytes: int = 80) -> int:
    f = lib().tq_pages_packed_bytes_for_slot
    f.restype = ctypes.c_size_t
    return f(ctypes.c_int(n_pages), ctypes.c_int(block_size), ctypes.c_int(num_kv_heads), ctypes.c_int(slot_bytes))


def _pages_args(kv_cache, page_ids, packed):
    for t, n in ((kv_cache, "kv_cache"), (page_ids, "page_ids"), (packed, "packed")):
        _cuda(t, n)
    if kv_cache.dim() != 5 or kv_cache.shape[0] != 2 or not kv_cache.is_contiguous() or kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must be contiguous 1-byte [2, num_blocks, block_size, heads, slot_bytes]")
    if page_ids.dtype != torch.int32 or not page_ids.is_contiguous() or page_ids.dim() != 1:
        raise TurboQuantError("page_ids must be a contiguous 1-D int32 tensor")
    if packed.dtype != torch.uint8 or not packed.is_contiguous():
        raise TurboQuantError("packed must be a contiguous uint8 tensor")


def pages_gather(kv_cache, page_ids, packed):
    """Pages ``page_ids`` of ``kv_cache`` -> ``packed`` uint8 [n, 2, block_size, H, 68] (device)."""
    _pages_args(kv_cache, page_ids, packed)
    _, nb, bs, H, ebs = kv_cache.shape
    _check(lib().tq_pages_gather(_ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(H),
                                 ctypes.c_int(ebs), _ptr(page_ids), ctypes.c_int(page_ids.shape[0]), _ptr(packed),
                                 ctypes.c_size_t(packed.numel()), _stream(kv_cache)))
    return packed


def pages_scatter(kv_cache, page_ids, packed):
    """The reverse of ``pages_gather``: ``packed`` -> pages ``page_ids`` of ``kv_cache``."""
    _pages_args(kv_cache, page_ids, packed)
    _, nb, bs, H, ebs = kv_cache.shape
    _check(lib().tq_pages_scatter(_ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(H),
                                  ctypes.c_int(ebs), _ptr(page_ids), ctypes.c_int(page_ids.shape[0]), _ptr(packed),
                                  ctypes.c_size_t(packed.numel()), _stream(kv_cache)))
    return kv_cache


def exchange_bytes(rows: int, world: int) -> int:
    """Bytes of one rank's exchange buffer for ``rows`` output rows (batch x queries x heads)."""
    f = lib().tq_exchange_bytes
    f.restype = ctypes.c_size_t
    n = f(ctypes.c_int64(rows), ctypes.c_int(world))
    if n == 0:
        raise TurboQuantError(f"exchange of {rows} rows over {world} ranks is not supported")
    return n


def decode_paged_exchange(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, workspace, rank: int,
                          exchange_ptrs, exchange_nbytes: int, out, page_indptr=None,
                          max_pages: int | None = None, out_lse=None, num_ctas: int = 0,
                          kv_begin: int = 0, kv_end: int = -1):
    """Decode this rank's KV range of a sequence split over ``len(exchange_ptrs)`` GPUs, exchange the
    partials through the ranks' mapped buffers and finish; ``q``/``out`` [batch, queries, Hq, D]."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    if q.dim() != 4 or not q.is_contiguous():
        raise TurboQuantError("q must be contiguous [batch, queries, num_q_heads, head_dim]")
    _decode_args(q.view(q.shape[0], -1, q.shape[3]), kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, NQ, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    world = len(exchange_ptrs)
    arr = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in exchange_ptrs])
    _check(lib().tq_decode_paged_exchange(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(NQ), ctypes.c_int(Hq),
        ctypes.c_int(H), ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens),
        ctypes.c_int64(kv_begin), ctypes.c_int64(kv_end), _ptr(signs), ctypes.c_float(sm_scale),
        _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        ctypes.c_int(rank), ctypes.c_int(world), arr, ctypes.c_size_t(exchange_nbytes),
        _ptr(out), ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse), ctypes.c_int(num_ctas), _stream(q)))
    return out


def decode_paged_partial(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, workspace,
                         out_rot, out_lse2, kv_begin: int = 0, kv_end: int = -1, page_indptr=None,
                         max_pages: int | None = None, num_ctas: int = 0):
    """Rotated-domain partial (fp32) + base-2 LSE over tokens [kv_begin, kv_end) of each sequence."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    _decode_args(q, kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    _check_rotated_partial(out_rot, D)
    _check(lib().tq_decode_paged_partial(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(H),
        ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens),
        ctypes.c_int64(kv_begin), ctypes.c_int64(kv_end), _ptr(signs), ctypes.c_float(sm_scale),
        _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        _ptr(out_rot), _ptr(out_lse2), ctypes.c_int(num_ctas), _stream(q)))
    return out_rot, out_lse2


def merge_rotated(partial_o, partial_lse2, signs, out, out_lse=None):
    """partial_o fp32 [parts, rows..., padded], partial_lse2 fp32 [parts, rows...] -> out [rows..., head_dim]
    (padded = 128 for head sizes 128 / 96, else 64, 128 or 256)."""
    _cuda(partial_o, "partial_o")
    _cuda(partial_lse2, "partial_lse2")
    if partial_o.dtype != torch.float32 or partial_lse2.dtype != torch.float32:
        raise TurboQuantError("partials must be fp32")
    parts = partial_o.shape[0]
    rows = partial_lse2.numel() // parts
    _check(lib().tq_merge_rotated(
        _ptr(partial_o.contiguous()), _ptr(partial_lse2.contiguous()), ctypes.c_int(parts),
        ctypes.c_int64(rows), ctypes.c_int(out.shape[-1]), _ptr(signs), _ptr(out),
        ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse), _stream(partial_o)))
    return out


def set_decode_events(ev_start=None, ev_mid=None, ev_end=None) -> None:
    """Measurement hook: torch.cuda.Event objects (created with enable_timing=True and recorded
    once so that their handle exists) recorded around the decode and merge kernels; None = off."""
    def h(e):
        return ctypes.c_void_p(0 if e is None else e.cuda_event)
    _check(lib().tq_debug_set_decode_events(h(ev_start), h(ev_mid), h(ev_end)))


def decode_paged_static(q, kv_cache, page_indices, seq_lens, signs, sm_scale: float, out,
                        page_indptr=None, max_pages: int | None = None, out_lse=None, num_ctas: int = 0):
    """``decode_paged`` for callers that may not allocate: the split-KV scratch is the fixed array
    built into the library (8 MiB per GPU), so no workspace tensor is passed.  Raises when the call
    would need more scratch than that.  Calls on one device share the array and must not overlap."""
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    _decode_args(q, kv_cache, page_indices, page_indptr, max_pages, seq_lens, signs)
    B, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    _check(lib().tq_decode_paged_static(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(H),
        ctypes.c_int(D), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(ebs),
        _ptr(page_indices), _ptr(page_indptr), ctypes.c_int(max_pages), _ptr(seq_lens), _ptr(signs),
        ctypes.c_float(sm_scale), _ptr(out), ctypes.c_int(dtype_code(out.dtype)), _ptr(out_lse),
        ctypes.c_int(num_ctas), _stream(q)))
    return out


def decode_static_status(device=None) -> int:
    """Sticky status word of the built-in scratch of ``decode_paged_static`` on the current device
    (0 = every call so far wrote all its partials); synchronises the current stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib().tq_decode_static_status(_ptr(word), _stream(word)))
    return int(word.item())


# ---- the slot format of vLLM's native backend ("turboquant_4bit_nc"): one cache tensor ------------
def nc_slot_bytes(head_dim: int) -> int:
    n = int(lib().tq_nc_slot_bytes(ctypes.c_int(head_dim)))
    if n == 0:
        raise TurboQuantError(f"head_dim {head_dim}: the upstream slot format takes 64, 128 or 256")
    return n


def nc_write_kv_cache(key, value, kv_cache, slot_mapping) -> None:
    """key / value [T, H, d] (fp32 / fp16 / bf16, last two dims contiguous) into kv_cache uint8
    [num_blocks, block_size, H, slot]; slot_mapping int32 / int64 [T], negative ids skipped."""
    for t, n in ((key, "key"), (value, "value"), (kv_cache, "kv_cache"), (slot_mapping, "slot_mapping")):
        _cuda(t, n)
    if key.dim() != 3 or key.shape != value.shape or key.dtype != value.dtype:
        raise TurboQuantError("key and value must both be [tokens, kv_heads, head_dim] of one dtype")
    if key.stride(2) != 1 or value.stride(2) != 1 or key.stride(1) != key.shape[2] or value.stride(1) != value.shape[2]:
        raise TurboQuantError("key / value: the last two dims must be contiguous")
    if kv_cache.dim() != 4 or not kv_cache.is_contiguous() or kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must be contiguous 1-byte [num_blocks, block_size, kv_heads, slot_bytes]")
    if slot_mapping.dtype not in (torch.int32, torch.int64) or not slot_mapping.is_contiguous():
        raise TurboQuantError("slot_mapping must be contiguous int32 or int64")
    T, H, D = key.shape
    nb, bs, Hc, sb = kv_cache.shape
    if Hc != H or slot_mapping.numel() < T:
        raise TurboQuantError("kv_cache heads / slot_mapping length do not match key")
    _check(lib().tq_nc_write_kv_cache(
        _ptr(key), _ptr(value), ctypes.c_int(dtype_code(key.dtype)), ctypes.c_int64(T), ctypes.c_int(H), ctypes.c_int(D),
        ctypes.c_int64(key.stride(0)), ctypes.c_int64(value.stride(0)), _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs),
        ctypes.c_int(sb), _ptr(slot_mapping), ctypes.c_int(1 if slot_mapping.dtype == torch.int64 else 0), _stream(key)))


def nc_decode_workspace_bytes(batch: int, num_q_heads: int, num_kv_heads: int, head_dim: int, num_ctas: int = 0) -> int:
    lib().tq_nc_decode_workspace_bytes.restype = ctypes.c_size_t
    return int(lib().tq_nc_decode_workspace_bytes(ctypes.c_int(batch), ctypes.c_int(num_q_heads), ctypes.c_int(num_kv_heads),
                                                  ctypes.c_int(head_dim), ctypes.c_int(num_ctas)))


def nc_decode_paged(q, kv_cache, page_indices, seq_lens, sm_scale: float, workspace, out, page_indptr=None,
                    max_pages: int | None = None, out_lse=None, num_ctas: int = 0):
    """One decode step over a cache in the upstream slot format: q / out [batch, Hq, d]."""
    for t, n in ((q, "q"), (kv_cache, "kv_cache"), (page_indices, "page_indices"), (seq_lens, "seq_lens"),
                 (workspace, "workspace"), (out, "out")):
        _cuda(t, n)
    if q.dim() != 3 or not q.is_contiguous() or out.shape != q.shape or not out.is_contiguous():
        raise TurboQuantError("q and out must be contiguous [batch, num_q_heads, head_dim]")
    if kv_cache.dim() != 4 or not kv_cache.is_contiguous() or kv_cache.element_size() != 1:
        raise TurboQuantError("kv_cache must be contiguous 1-byte [num_blocks, block_size, kv_heads, slot_bytes]")
    for t, n in ((page_indices, "page_indices"), (seq_lens, "seq_lens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise TurboQuantError(f"{n} must be contiguous int32")
    if max_pages is None:
        max_pages = page_indices.shape[-1] if page_indices.dim() == 2 else 0
    B, Hq, D = q.shape
    nb, bs, H, sb = kv_cache.shape
    _check(lib().tq_nc_decode_paged(
        _ptr(q), ctypes.c_int(dtype_code(q.dtype)), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(H), ctypes.c_int(D),
        _ptr(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(sb), _ptr(page_indices), _ptr(page_indptr),
        ctypes.c_int(max_pages), _ptr(seq_lens), ctypes.c_float(sm_scale), _ptr(workspace),
        ctypes.c_size_t(workspace.numel() * workspace.element_size()), _ptr(out), ctypes.c_int(dtype_code(out.dtype)),
        _ptr(out_lse), ctypes.c_int(num_ctas), _stream(q)))
    return out


def nc_write_dropped() -> int:
    n = ctypes.c_int32(0)
    _check(lib().tq_nc_write_dropped(ctypes.byref(n)))
    return int(n.value)
