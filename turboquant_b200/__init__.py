"""B200-native TurboQuant KV-cache hot paths (cache write + paged decode attention), behind the
interface of RRoundTable/turboquant: ``TurboQuantMSE``, ``RandomHadamardRotation``, ``Codebook``,
``fwht`` and the CUSTOM vLLM backend (``turboquant_b200.vllm_backend_fused``)."""
__version__ = "0.1.0"

_LAZY = {
    "TurboQuantMSE": ("quantizer", "TurboQuantMSE"),
    "RandomHadamardRotation": ("hadamard", "RandomHadamardRotation"),
    "fwht": ("hadamard", "fwht"),
    "Codebook": ("codebook", "Codebook"),
    "TurboQuantPagedAttention": ("paged_attention", "TurboQuantPagedAttention"),
}
__all__ = sorted(_LAZY)


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(name)
