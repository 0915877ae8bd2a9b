"""vLLM plugin entry point, ``vllm.general_plugins: turboquant_b200 = turboquant_b200.vllm_plugin:register``
(the reference's is turboquant/vllm_plugin.py:85-92 with pyproject.toml:20-21).

``register()`` binds ``turboquant_b200.vllm_backend_fused.TurboQuantBackend`` to
``AttentionBackendEnum.CUSTOM`` so that ``--attention-backend CUSTOM --kv-cache-dtype fp8`` selects
it.  (The reference archived this registration when it moved to patching upstream Triton kernels;
nothing is patched here.)
"""
from __future__ import annotations

_registered = False
BACKEND_PATH = "turboquant_b200.vllm_backend_fused.TurboQuantBackend"


def register() -> None:
    """Called once per process at vLLM start-up; registering twice is a no-op."""
    global _registered
    if _registered:
        return
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_PATH)
    _registered = True
