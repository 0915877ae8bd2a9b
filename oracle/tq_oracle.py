"""ctypes front-end of the CPU oracle (oracle/tq_oracle.c).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is the
checker used by tests/, by the smoke check and by the benchmark's CPU-baseline leg.

All tensors cross this boundary as C-contiguous numpy arrays.  Inputs in bf16/fp16 are
widened to fp32 by the caller (exactly representable), as the reference does with
``key.float()`` before quantizing (turboquant/vllm_backend_fused.py:301).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libtq_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile the C restatement (and, when TURBOQUANT_REFERENCE names the reference tree, its pack.cpp)."""
    src = _HERE / "tq_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["make", "-C", str(_HERE), "-B", "libtq_oracle.so"],
                              stdout=subprocess.DEVNULL)
    ref = os.environ.get("TURBOQUANT_REFERENCE", "")
    if ref and os.path.isdir(ref) and not (_HERE / "_ref" / "libref_pack.so").exists():
        subprocess.call(["make", "-C", str(_HERE), "ref", f"REF={ref}"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.tqo_f16_to_f32.restype = ctypes.c_float
        _lib.tqo_f32_to_f16.restype = ctypes.c_uint16
        _lib.tqo_f32_to_f16.argtypes = [ctypes.c_float]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def codebook(dim: int, bits: int = 4):
    cen = np.zeros(1 << bits, np.float32)
    bnd = np.zeros((1 << bits) - 1, np.float32)
    lib().tqo_codebook(ctypes.c_int(dim), ctypes.c_int(bits), _p(cen), _p(bnd))
    return cen, bnd


def fwht(x) -> np.ndarray:
    x = _f32(x).copy()
    d = x.shape[-1]
    flat = x.reshape(-1, d)
    for r in range(flat.shape[0]):
        row = np.ascontiguousarray(flat[r])
        lib().tqo_fwht(_p(row), ctypes.c_int(d))
        flat[r] = row
    return flat.reshape(x.shape)


def quantize_flat(x, signs, bits: int = 4):
    """TurboQuantMSE.quantize: (packed uint8 [..., nbytes] low-first order, norms fp32 [...])."""
    x = _f32(x)
    d = x.shape[-1]
    padded = next_pow2(d)
    n = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
    vpb = 8 // bits
    nbytes = (padded + vpb - 1) // vpb
    packed = np.zeros((n, nbytes), np.uint8)
    norms = np.zeros(n, np.float32)
    lib().tqo_quantize_flat(_p(x), ctypes.c_int64(n), ctypes.c_int(d), ctypes.c_int(padded),
                            _p(_f32(signs)), ctypes.c_int(bits), _p(packed), _p(norms))
    return packed.reshape(x.shape[:-1] + (nbytes,)), norms.reshape(x.shape[:-1])


def dequantize_flat(packed, norms, signs, dim: int, bits: int = 4) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint8)
    norms = _f32(norms)
    n = int(np.prod(norms.shape)) if norms.ndim else 1
    padded = next_pow2(dim)
    out = np.zeros((n, dim), np.float32)
    lib().tqo_dequantize_flat(_p(packed), _p(norms), ctypes.c_int64(n), ctypes.c_int(dim),
                              ctypes.c_int(padded), _p(_f32(signs)), ctypes.c_int(bits), _p(out))
    return out.reshape(norms.shape + (dim,))


def write_kv_cache(kv_cache: np.ndarray, key, value, signs, slot_mapping, head_dim: int,
                   token_stride: int | None = None) -> None:
    """In-place paged write.  kv_cache: uint8 [2, num_blocks, block_size, H, ebs];
    key/value: fp32 [T, H, head_dim] (or a flat buffer with ``token_stride`` floats per token)."""
    assert kv_cache.dtype == np.uint8 and kv_cache.flags.c_contiguous and kv_cache.shape[0] == 2
    _, nb, bs, H, ebs = kv_cache.shape
    key, value = _f32(key), _f32(value)
    slots = np.ascontiguousarray(slot_mapping, np.int64)
    T = slots.shape[0]
    if token_stride is None:
        token_stride = H * head_dim
    lib().tqo_write_kv_cache(_p(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs), ctypes.c_int(H),
                             ctypes.c_int(ebs), _p(key), _p(value), ctypes.c_int64(T),
                             ctypes.c_int64(token_stride), _p(_f32(signs)), _p(slots),
                             ctypes.c_int(head_dim))


def dequant_cache_rows(slots: np.ndarray, signs, head_dim: int) -> np.ndarray:
    """slots: uint8 [..., ebs] -> fp32 [..., head_dim] un-rotated dequantized vectors."""
    slots = np.ascontiguousarray(slots, np.uint8)
    ebs = slots.shape[-1]
    n = int(np.prod(slots.shape[:-1]))
    out = np.zeros((n, head_dim), np.float32)
    lib().tqo_dequant_cache_rows(_p(slots), ctypes.c_int64(n), ctypes.c_int(ebs),
                                 ctypes.c_int(head_dim), _p(_f32(signs)), _p(out))
    return out.reshape(slots.shape[:-1] + (head_dim,))


def decode_paged(q, kv_cache: np.ndarray, block_table, seq_lens, signs, sm_scale: float,
                 kv_begin: int = 0, kv_end: int = -1, return_lse: bool = False):
    """One decode step.  q fp32 [B, Hq, D]; returns out fp32 [B, Hq, D] (and natural-log lse)."""
    q = _f32(q)
    B, Hq, D = q.shape
    _, nb, bs, H, ebs = kv_cache.shape
    bt = np.ascontiguousarray(block_table, np.int32)
    sl = np.ascontiguousarray(seq_lens, np.int32)
    out = np.zeros((B, Hq, D), np.float32)
    lse = np.zeros((B, Hq), np.float32)
    lib().tqo_decode_paged(_p(q), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(H),
                           ctypes.c_int(D), _p(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs),
                           ctypes.c_int(ebs), _p(bt), ctypes.c_int(bt.shape[1]), _p(sl),
                           _p(_f32(signs)), ctypes.c_float(sm_scale), ctypes.c_int64(kv_begin),
                           ctypes.c_int64(kv_end), _p(out), _p(lse))
    return (out, lse) if return_lse else out


def decode_paged_parallel(q, kv_cache: np.ndarray, block_table, seq_lens, signs, sm_scale: float,
                          threads: int | None = None, chunk_tokens: int = 8192, return_lse: bool = False):
    """``decode_paged`` at benchmark sizes: every sequence's token range is cut into chunks of
    ``chunk_tokens``, the chunks run on ``threads`` host threads (the C call releases the GIL) and
    the per-chunk (out, lse) pairs are combined with ``merge_partials``.  Same arithmetic per
    chunk as ``decode_paged``; the merge is the log-sum-exp identity in double precision."""
    from concurrent.futures import ThreadPoolExecutor
    q = _f32(q)
    B, Hq, D = q.shape
    bt = np.ascontiguousarray(block_table, np.int32)
    sl = np.ascontiguousarray(seq_lens, np.int32)
    threads = threads or os.cpu_count() or 1
    jobs = []
    for b in range(B):
        n = int(sl[b])
        cuts = list(range(0, n, chunk_tokens)) or [0]
        for a in cuts:
            jobs.append((b, a, min(a + chunk_tokens, n)))

    def one(job):
        b, a, e = job
        return decode_paged(q[b:b + 1], kv_cache, bt[b:b + 1], sl[b:b + 1], signs, sm_scale,
                            kv_begin=a, kv_end=max(e, a), return_lse=True)
    lib()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        parts = list(ex.map(one, jobs))
    out = np.zeros((B, Hq, D), np.float32)
    lse = np.full((B, Hq), -np.inf, np.float32)
    for b in range(B):
        mine = [p for j, p in zip(jobs, parts) if j[0] == b]
        po = np.stack([p[0][0] for p in mine])
        pl = np.stack([p[1][0] for p in mine])
        out[b], lse[b] = merge_partials(po, pl)
    return (out, lse) if return_lse else out


def merge_partials(partial_o, partial_lse):
    """partial_o fp32 [S, rows..., D], partial_lse fp32 [S, rows...] (natural log)."""
    po, pl = _f32(partial_o), _f32(partial_lse)
    S, D = po.shape[0], po.shape[-1]
    rows = int(np.prod(pl.shape[1:]))
    out = np.zeros((rows, D), np.float32)
    lse = np.zeros(rows, np.float32)
    lib().tqo_merge_partials(_p(po), _p(pl), ctypes.c_int(S), ctypes.c_int64(rows),
                             ctypes.c_int(D), _p(out), _p(lse))
    return out.reshape(pl.shape[1:] + (D,)), lse.reshape(pl.shape[1:])


def pack_4bit_cache_order(idx: np.ndarray) -> np.ndarray:
    """Cache nibble order: byte = (idx[2i] << 4) | idx[2i+1] (turboquant/tile.py:37-41)."""
    idx = np.asarray(idx, np.uint8)
    return ((idx[..., 0::2] << 4) | (idx[..., 1::2] & 0x0F)).astype(np.uint8)


def low_first_to_cache_order(packed: np.ndarray) -> np.ndarray:
    """Swap nibbles: TurboQuantMSE's _pack_bits order -> the paged cache's order."""
    packed = np.asarray(packed, np.uint8)
    return (((packed & 0x0F) << 4) | (packed >> 4)).astype(np.uint8)


# ---------------------------------------------------------------------------------------------
# The slot format of vLLM's native backend ("turboquant_4bit_nc"), restated from the description
# in docs/reference/vllm-upstream-turboquant-architecture.md:33-94 (layout), :100-175 (store),
# :178-240 (decode).  PARITY UNPINNED: the reference tree has neither code nor vectors for it.
# ---------------------------------------------------------------------------------------------
def nc_slot_bytes(head_dim: int) -> int:
    return (head_dim // 2 + 2) + (head_dim // 2 + 4)


def nc_store(kv_cache: np.ndarray, key, value, slot_mapping) -> None:
    """kv_cache uint8 [nb, bs, H, slot]; key / value [T, H, d] (values as the kernel sees them after
    the cast to fp32); slots with a negative id are skipped."""
    key, value = _f32(key), _f32(value)
    T, H, d = key.shape
    nb, bs, _, sb = kv_cache.shape
    rows = np.zeros((T * H, sb), np.uint8)
    L = lib()
    L.tqo_nc_store_rows.restype = None
    L.tqo_nc_store_rows(_p(key.reshape(T * H, d)), _p(value.reshape(T * H, d)), ctypes.c_int64(T * H), ctypes.c_int(d),
                        _p(rows), ctypes.c_int(sb))
    rows = rows.reshape(T, H, sb)
    flat = kv_cache.reshape(nb * bs, H, sb)
    n = nc_slot_bytes(d)
    for t, s in enumerate(np.asarray(slot_mapping).tolist()):
        if s >= 0:
            flat[s, :, :n] = rows[t, :, :n]


def nc_decode(q, kv_cache: np.ndarray, block_table, seq_lens, sm_scale: float, return_lse: bool = False):
    """q [B, Hq, d] -> out [B, Hq, d]: scores in the rotated domain (q H / sqrt(d) against the K
    centroids times the fp16 norm), values code * scale + zero, fp32 softmax."""
    q = _f32(q)
    B, Hq, d = q.shape
    nb, bs, H, sb = kv_cache.shape
    g = Hq // H
    cen, _ = codebook(d, 4)
    qb, kps = d // 2, d // 2 + 2
    out = np.zeros((B, Hq, d), np.float32)
    lse = np.full((B, Hq), -np.inf, np.float32)
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            continue
        t = np.arange(n)
        slots = kv_cache[np.asarray(block_table)[b, t // bs], t % bs]          # [n, H, sb]
        kc = slots[..., :qb]
        kidx = np.stack((kc & 15, kc >> 4), -1).reshape(n, H, d)
        kn = slots[..., qb:qb + 2].copy().view(np.float16).astype(np.float32)[..., 0]
        khat = cen[kidx] * kn[..., None]
        vc = slots[..., kps:kps + qb]
        vidx = np.stack((vc & 15, vc >> 4), -1).reshape(n, H, d).astype(np.float32)
        vsz = slots[..., kps + qb:kps + qb + 4].copy().view(np.float16).astype(np.float32)   # [n, H, 2]
        vhat = vidx * vsz[..., :1] + vsz[..., 1:]
        qr = fwht(q[b].reshape(Hq, d)).reshape(H, g, d)
        s = np.einsum("hgd,nhd->hgn", qr, khat).astype(np.float64) * sm_scale
        m = s.max(-1, keepdims=True)
        e = np.exp(s - m)
        l = e.sum(-1, keepdims=True)
        out[b] = np.einsum("hgn,nhd->hgd", e / l, vhat.astype(np.float64)).reshape(Hq, d).astype(np.float32)
        lse[b] = (m + np.log(l)).reshape(Hq).astype(np.float32)
    return (out, lse) if return_lse else out
