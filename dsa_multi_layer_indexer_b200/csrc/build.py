"""Builds libdsa_b200.so in-tree with nvcc for sm_100a.

Run as ``python -m dsa_multi_layer_indexer_b200.csrc.build`` or call
:func:`build`. nvcc cross-compiles without a GPU, so this also works on a
CPU-only machine. The library is rebuilt only when a source is newer than it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB = PKG / "libdsa_b200.so"
SOURCES = ["dsa_b200.cu"]
HEADERS = ["common.cuh", "indexer_scan.cuh", "topk_select.cuh", "sparse_mla.cuh", "sparse_mla_tc.cuh",
           "fused_decode.cuh", "decode_prep.cuh", "peer_allreduce.cuh"]
PUBLIC_HEADER = PKG.parent / "include" / "dsa_b200.h"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = [CSRC / f for f in SOURCES + HEADERS] + [PUBLIC_HEADER]
    return any(d.stat().st_mtime > built for d in deps)


def build_trace(out: Path) -> Path:
    """Tracing build: same ABI plus per-CTA phase stamps (dsa_debug_read_stamps).
    Select it at run time with DSA_B200_LIB=<out>."""
    cmd = [_nvcc(), *NVCC_FLAGS, "-DDSA_STAMPS", "-o", str(out), *[str(CSRC / s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"nvcc failed ({proc.returncode})")
    return out


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB), *[str(CSRC / s) for s in SOURCES]]  # cudart is linked statically (nvcc default)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace(Path(sys.argv[sys.argv.index("--trace") + 1])))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
