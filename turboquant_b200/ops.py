"""Dispatcher-visible torch ops under the reference's names and schemas, implemented by the C ABI.

    torch.ops.turboquant_write.quantize_write_kv_cache      (csrc/src/quantize_write_binding.cu:284-286)
    torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws
    torch.ops.turboquant_v5.decode_v5_from_cache_ws          (csrc/src/decode_v5_tc_binding.cu:947-981)

``kv_cache`` is a mutable tensor argument, so the dispatcher refreshes its storage pointer on
CUDA-graph replay as with the reference's ops.  Only a CUDA implementation is registered: a CPU
tensor fails in the dispatcher (there is no fallback).  Importing this module registers the ops
once per process.
"""
from __future__ import annotations

import torch

from . import _cabi

_WRITE = torch.library.Library("turboquant_write", "DEF")
_V5 = torch.library.Library("turboquant_v5", "DEF")

_WRITE.define("quantize_write_kv_cache(Tensor(a!) kv_cache, Tensor key, Tensor value, Tensor signs, "
              "Tensor slot_mapping, int head_dim, int padded_dim) -> ()")
_V5.define("decode_v5_from_cache_paged_splitkv_ws(Tensor q, Tensor kv_cache, Tensor indices, Tensor indptr, "
           "Tensor last_page_len, Tensor seq_lens, int num_kv_heads, int page_size, int head_dim, int padded_dim, "
           "float sm_scale, Tensor hadamard_signs, int qbytes, int nbytes, Tensor(a!) o_ws, int max_len, "
           "Tensor partition_o_ws, Tensor partition_lse_ws, Tensor request_indices, Tensor kv_tile_indices, "
           "Tensor split_indptr, Tensor kv_chunk_size_t, int num_splits) -> Tensor(a!)")
_V5.define("decode_v5_from_cache_ws(Tensor q, Tensor kv_cache, Tensor indices, Tensor indptr, "
           "Tensor last_page_len, Tensor seq_lens, int num_kv_heads, int page_size, int head_dim, int padded_dim, "
           "float sm_scale, Tensor hadamard_signs, int qbytes, int nbytes, Tensor k_quant_ws, Tensor v_quant_ws, "
           "Tensor k_norms_ws, Tensor v_norms_ws, Tensor(a!) o_ws, int max_len) -> Tensor(a!)")

_workspaces: dict[tuple, torch.Tensor] = {}


def _bytes(kv_cache: torch.Tensor) -> torch.Tensor:
    return kv_cache if kv_cache.dtype == torch.uint8 else kv_cache.view(torch.uint8)


def _workspace(batch: int, hq: int, hkv: int, head_dim: int, device) -> torch.Tensor:
    key = (device.index, batch, hq, hkv, head_dim)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_cabi.decode_workspace_bytes(batch, hq, hkv, head_dim), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_dims(head_dim: int, padded_dim: int) -> None:
    """The reference pads the head to the next power of two, 64 at least (turboquant/vllm_backend_fused.py:28-29,
    64-72); its own decode op takes 128 only, the kernels here head sizes 33 ... 256."""
    want = max(64, 1 << (int(head_dim) - 1).bit_length()) if head_dim > 0 else 0
    if not 32 < head_dim <= 256 or padded_dim != want:
        raise _cabi.TurboQuantError(f"head_dim {head_dim} / padded_dim {padded_dim}: head sizes 33 ... 256 with the "
                                    f"next power of two (64 at least) as padded size are implemented")


def _quantize_write_kv_cache(kv_cache, key, value, signs, slot_mapping, head_dim, padded_dim):
    _check_dims(head_dim, padded_dim)
    _cabi.write_kv_cache(_bytes(kv_cache), key, value, signs, slot_mapping, head_dim)


def _decode(q, kv_cache, indices, indptr, seq_lens, num_kv_heads, page_size, head_dim, padded_dim, sm_scale,
            signs, o_ws):
    _check_dims(head_dim, padded_dim)
    b, hq, _ = q.shape
    # The op runs inside CUDA graphs: a silent cast or copy here would be an extra kernel and an
    # allocation on every replay.  The reference passes int32 tables and a contiguous q
    # (turboquant/vllm_backend_fused.py:396-402); anything else is refused.
    for t, name in ((indices, "indices"), (indptr, "indptr"), (seq_lens, "seq_lens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise _cabi.TurboQuantError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")
    if not q.is_contiguous():
        raise _cabi.TurboQuantError("q must be contiguous")
    ws = _workspace(b, hq, num_kv_heads, head_dim, q.device)
    _cabi.decode_paged(q, _bytes(kv_cache), indices, seq_lens, signs, float(sm_scale), ws, o_ws,
                       page_indptr=indptr, max_pages=1)
    return o_ws


def _decode_paged_splitkv_ws(q, kv_cache, indices, indptr, last_page_len, seq_lens, num_kv_heads, page_size,
                             head_dim, padded_dim, sm_scale, hadamard_signs, qbytes, nbytes, o_ws, max_len,
                             partition_o_ws, partition_lse_ws, request_indices, kv_tile_indices, split_indptr,
                             kv_chunk_size_t, num_splits):
    # The split plan is made on the device from seq_lens; the reference's split arguments and
    # partition workspaces are accepted for signature compatibility and not used.
    return _decode(q, kv_cache, indices, indptr, seq_lens, num_kv_heads, page_size, head_dim, padded_dim, sm_scale,
                   hadamard_signs, o_ws)


def _decode_ws(q, kv_cache, indices, indptr, last_page_len, seq_lens, num_kv_heads, page_size, head_dim,
               padded_dim, sm_scale, hadamard_signs, qbytes, nbytes, k_quant_ws, v_quant_ws, k_norms_ws,
               v_norms_ws, o_ws, max_len):
    # The reference gathers the pages into contiguous workspaces first; the paged kernel needs none.
    return _decode(q, kv_cache, indices, indptr, seq_lens, num_kv_heads, page_size, head_dim, padded_dim, sm_scale,
                   hadamard_signs, o_ws)


_WRITE.impl("quantize_write_kv_cache", _quantize_write_kv_cache, "CUDA")
_V5.impl("decode_v5_from_cache_paged_splitkv_ws", _decode_paged_splitkv_ws, "CUDA")
_V5.impl("decode_v5_from_cache_ws", _decode_ws, "CUDA")
