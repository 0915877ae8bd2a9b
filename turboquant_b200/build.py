"""Builds libturboquant_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m turboquant_b200.build [--force]

The cache-write, flat-quantizer and bulk-dequantizer translation units are compiled with -fmad=false: their
arithmetic must round every product and sum separately to stay bit-identical to the torch
quantizer.  No torch headers are involved; the library exports plain C symbols only.
"""
from __future__ import annotations

import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libturboquant_b200.so"
HEADER = PKG.parent / "include" / "turboquant_b200.h"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
UNITS = {
    "tq_api.cu": [],
    "tq_write.cu": ["-fmad=false"],
    "tq_flat.cu": ["-fmad=false"],
    "tq_decode.cu": [],
    "tq_decode_mq.cu": [],
    "tq_dequant.cu": ["-fmad=false"],
    "tq_pages.cu": [],
    "tq_generic.cu": ["-fmad=false"],
    "tq_nc.cu": ["-fmad=false"],
}


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def build(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    deps = [CSRC / "tq_common.cuh", CSRC / "tq_decode_common.cuh", HEADER, Path(__file__)]

    def compile_one(item):
        name, extra = item
        src, obj = CSRC / name, obj_dir / (name + ".o")
        if force or _stale(obj, [src, *deps]):
            cmd = ["nvcc", *ARCH, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, UNITS.items()))
    if force or _stale(LIB, objs):
        subprocess.check_call(["nvcc", *ARCH, "-shared", "-o", str(LIB), *map(str, objs)])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
