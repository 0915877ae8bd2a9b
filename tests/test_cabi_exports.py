"""The C-ABI library builds, loads and exports every symbol the public header declares
(no compute call is made here: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from turboquant_b200 import build
    return ctypes.CDLL(str(build.build()))


def declared_symbols():
    text = (ROOT / "include" / "turboquant_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_python_binding_lists_same_symbols():
    from turboquant_b200 import _cabi
    assert sorted(_cabi.EXPORTS) == declared_symbols()


def test_abi_version_and_codebook(lib, golden):
    assert lib.tq_abi_version() == 1
    from turboquant_b200 import _cabi
    import numpy as np
    for dim in (64, 128, 256):
        for bits in (1, 2, 3, 4):
            cen, bnd = _cabi.codebook(dim, bits)
            np.testing.assert_array_equal(cen.numpy(), golden[f"centroids_d{dim}_b{bits}"])
            np.testing.assert_array_equal(bnd.numpy(), golden[f"boundaries_d{dim}_b{bits}"])


def test_argument_errors_reported_without_gpu(lib):
    lib.tq_last_error.restype = ctypes.c_char_p
    rc = lib.tq_codebook(ctypes.c_int(128), ctypes.c_int(9), None, None)
    assert rc == 1 and b"null" in lib.tq_last_error()
    f = (ctypes.c_float * 16)()
    rc = lib.tq_codebook(ctypes.c_int(128), ctypes.c_int(9), f, f)
    assert rc == 1 and b"bits" in lib.tq_last_error()
    # null pointers are rejected before any CUDA call
    rc = lib.tq_write_kv_cache(None, ctypes.c_int64(1), 16, 8, 80, None, None, 2, ctypes.c_int64(4),
                               ctypes.c_int64(1024), ctypes.c_int64(1024), None, None, 1, 128, 0, None)
    assert rc == 1
    rc = lib.tq_decode_paged(None, 1, 2, 32, 8, 128, None, ctypes.c_int64(4), 16, 80, None, None, 4, None,
                             None, ctypes.c_float(0.1), None, ctypes.c_size_t(0), None, 1, None, 0, None)
    assert rc == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from turboquant_b200 import _cabi
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_cabi.TurboQuantError, match="no CPU or PyTorch fallback"):
        _cabi.lib()


def test_cpu_tensors_rejected():
    import torch
    from turboquant_b200 import _cabi
    with pytest.raises(_cabi.TurboQuantError, match="CUDA tensor"):
        _cabi.quantize_flat(torch.zeros(2, 128), torch.ones(128), 4)
