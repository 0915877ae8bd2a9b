"""Model geometry presets and the launch geometry of the sm_100a decode kernel.

Keeps the reference's ``ModelConfig`` / ``KernelConfig`` / ``compute_kernel_config`` /
``MODEL_PRESETS`` names (turboquant/kernel_config.py:10-109).  The reference's fields described a
(bdx, bdy, bdz) thread block of its scalar v4 kernel; here a config describes the one-block-per-SM
streaming kernel: warps per block, pages per stage and ring depth, all derived from the head
geometry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

CONSUMER_WARPS = 16
PAGE_TOKENS = 16
SLOT_BYTES = 80
MAX_SMEM = 227 * 1024


@dataclass(frozen=True)
class ModelConfig:
    num_qo_heads: int
    num_kv_heads: int
    head_dim: int
    name: str = ""

    @property
    def gqa_ratio(self) -> int:
        return self.num_qo_heads // self.num_kv_heads

    @property
    def padded_dim(self) -> int:
        return ((self.head_dim + 63) // 64) * 64


@dataclass(frozen=True)
class KernelConfig:
    """Geometry of ``decode_paged_kernel``: one block of ``threads_per_block`` threads per SM."""
    consumer_warps: int
    pages_per_stage: int
    stages: int
    stage_bytes: int
    supported: bool = True
    reason: str = ""
    tuned: bool = True    # False: the second-tier kernels for head sizes other than 128 / 96

    @property
    def threads_per_block(self) -> int:
        # consumer warps + a producer warpgroup (the producer warp and three register donors)
        return (self.consumer_warps + 4) * 32

    @property
    def tile_tokens(self) -> int:
        return self.pages_per_stage * PAGE_TOKENS


def compute_kernel_config(model: ModelConfig, max_threads: int = 1024) -> KernelConfig:
    h, g = model.num_kv_heads, model.gqa_ratio
    if model.head_dim not in (128, 96):
        if 32 < model.head_dim <= 256 and 1 <= g <= 8:
            # four warps per (split, sequence, KV head), each with its own ring of one-page stages
            pd = 64 if model.head_dim <= 64 else 128 if model.head_dim <= 128 else 256
            row = (pd // 2 + 2 * (pd // 64) + 15) & ~15
            return KernelConfig(4, 1, 2 if pd == 256 else 3, 2 * PAGE_TOKENS * row, True,
                                "second-tier kernels (head sizes other than 128 / 96: 25 - 40 % of the HBM peak)", False)
        return KernelConfig(CONSUMER_WARPS, 0, 0, 0, False,
                            f"head_dim {model.head_dim} with GQA ratio {g}: head sizes 33..256 and ratios 1..8 are implemented")
    if h not in (1, 2, 4, 8, 16):
        if h > 8 and h % 4 == 0:
            # several launches of 16, 8 or 4 heads on strided token rows (one copy per token row)
            c = 16 if h >= 16 else 8
            row = c * SLOT_BYTES
            kp, vp = row + (64 - row % 128) % 128, row + (16 - row % 128) % 128
            return KernelConfig(CONSUMER_WARPS, CONSUMER_WARPS // c, 3, (CONSUMER_WARPS // c) * PAGE_TOKENS * (kp + vp))
        return KernelConfig(CONSUMER_WARPS, 0, 0, 0, False, f"{h} KV heads per GPU: 1, 2, 4, 8, 16 or a larger multiple of 4")
    if not 1 <= g <= 8:
        return KernelConfig(CONSUMER_WARPS, 0, 0, 0, False, f"GQA ratio {g}: 1..8 is implemented")
    pps = CONSUMER_WARPS // h
    # per page lane: K region + V region (runs of token rows, placed for conflict-free fragment loads)
    stage = pps * {16: 20736 + 20736, 8: 10496 + 10368, 4: 5248 + 5248, 2: 2560 + 2560, 1: 1280 + 1280}[h]
    # lookup table (256 B per entry, per-warp scratch in the unused halves) at the 64 KB boundary of
    # the shared window; three stages: one below the table and two above it
    return KernelConfig(CONSUMER_WARPS, pps, 3, stage)


MODEL_PRESETS: Dict[str, ModelConfig] = {
    "llama-2-7b": ModelConfig(32, 32, 128, "Llama-2-7B"),
    "llama-2-13b": ModelConfig(40, 40, 128, "Llama-2-13B"),
    "llama-2-70b": ModelConfig(64, 8, 128, "Llama-2-70B"),
    "llama-3-8b": ModelConfig(32, 8, 128, "Llama-3-8B"),
    "llama-3-70b": ModelConfig(64, 8, 128, "Llama-3-70B"),
    "llama-3.1-8b": ModelConfig(32, 8, 128, "Llama-3.1-8B"),
    "llama-3.1-70b": ModelConfig(64, 8, 128, "Llama-3.1-70B"),
    "qwen3-0.6b": ModelConfig(16, 8, 64, "Qwen3-0.6B"),
    "qwen3-1.7b": ModelConfig(16, 8, 128, "Qwen3-1.7B"),
    "qwen3-4b": ModelConfig(32, 8, 128, "Qwen3-4B"),
    "qwen3-8b": ModelConfig(32, 8, 128, "Qwen3-8B"),
    "qwen3-14b": ModelConfig(40, 8, 128, "Qwen3-14B"),
    "qwen3-32b": ModelConfig(40, 8, 128, "Qwen3-32B"),
    "mistral-7b": ModelConfig(32, 8, 128, "Mistral-7B"),
    "mixtral-8x7b": ModelConfig(32, 8, 128, "Mixtral-8x7B"),
    "mistral-nemo": ModelConfig(32, 8, 128, "Mistral-Nemo-12B"),
    "phi-3-mini": ModelConfig(32, 32, 96, "Phi-3-mini"),
    "phi-3-small": ModelConfig(32, 8, 96, "Phi-3-small"),
    "gemma-2-2b": ModelConfig(8, 4, 256, "Gemma-2-2B"),
    "gemma-2-9b": ModelConfig(16, 8, 256, "Gemma-2-9B"),
    "yi-6b": ModelConfig(32, 4, 128, "Yi-6B"),
    "yi-34b": ModelConfig(56, 8, 128, "Yi-34B"),
}
