"""Decode-op selection with the reference's interface (turboquant/decoder_dispatch.py:83-139).

The reference picks one of several kernel generations by compute capability.  This library has
exactly one decode kernel, written for sm_100a, so ``pick_decode_op`` returns it or raises: there
is no multi-backend dispatch and no fallback.
"""
from __future__ import annotations

import os
from functools import lru_cache

import torch

KERNEL_NAME = "b200_paged_split_sm100a"


@lru_cache(maxsize=1)
def _device_capability() -> tuple[int, int]:
    if not torch.cuda.is_available():
        return (0, 0)
    return torch.cuda.get_device_capability()


def _op():
    from . import ops  # noqa: F401  (registers torch.ops.turboquant_v5.*)
    return torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws


@lru_cache(maxsize=1)
def pick_decode_op():
    """Return ``(op_callable, kernel_name)``; the op has the reference's unified signature."""
    forced = os.environ.get("TQ_FORCE_KERNEL", "").strip().lower()
    if forced and forced not in ("b200", "v7", KERNEL_NAME):
        raise ValueError(f"TQ_FORCE_KERNEL={forced!r} not recognised: this build has the single kernel "
                         f"{KERNEL_NAME!r} (aliases 'b200', 'v7')")
    cc = _device_capability()
    if cc < (10, 0):
        raise RuntimeError(f"compute capability {cc} is not supported: the kernels are built for sm_100a only")
    if os.environ.get("TQ_DEBUG_KERNEL"):
        print(f"[TQ dispatch] cc={cc} -> {KERNEL_NAME}", flush=True)
    return _op(), KERNEL_NAME
