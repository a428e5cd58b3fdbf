"""Recipe for ``oracle/_ref``: the reference's own CPU implementation of the path.

The reference is pure Python. Its decode-form CPU functions live in two places:
the package ``src/lagged_indexer_dsa`` (``attention_core.indexer_logits``,
``select_topk``, ``_attend`` ...) and the host helpers at the bottom of
``kernels/cuda_fused_sparse_splitk.py`` (``ref_indexer_logits_fp8`` :2990-2992,
``ref_sparse_mla`` :2950-2966, ``quantize_e4m3_rowwise`` :2969-2974), which import
the package at module level (:36-37). This recipe places an unmodified copy of
both under ``oracle/_ref/`` so that they can be imported on a machine that has no
reference checkout. ``oracle/_ref/`` is listed in ``.gitignore``: the copy is a
build output, never part of this repository's history.

    python -m oracle.build_ref [/path/to/reference]

Test infrastructure only: nothing in the product imports ``oracle``.
"""

from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
DEFAULT_REFERENCE = Path("/root/reference")


def build_ref(reference: Path = DEFAULT_REFERENCE) -> Path | None:
    """Copies the two pieces named above into ``oracle/_ref``; returns the folder,
    or None when there is no reference checkout (the prebuilt folder, if any, stays)."""
    pkg = reference / "src" / "lagged_indexer_dsa"
    kern = reference / "kernels" / "cuda_fused_sparse_splitk.py"
    if not pkg.is_dir() or not kern.is_file():
        return REF_OUT if (REF_OUT / "cuda_fused_sparse_splitk.py").exists() else None
    REF_OUT.mkdir(exist_ok=True)
    dst_pkg = REF_OUT / "lagged_indexer_dsa"
    if dst_pkg.exists():
        shutil.rmtree(dst_pkg)
    shutil.copytree(pkg, dst_pkg, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    shutil.copyfile(kern, REF_OUT / kern.name)
    return REF_OUT


def load_ref():
    """The reference's kernel-file module (with its host-side reference functions)
    imported from ``oracle/_ref``, or None when that folder was never built."""
    if not (REF_OUT / "cuda_fused_sparse_splitk.py").exists():
        return None
    if str(REF_OUT) not in sys.path:
        sys.path.insert(0, str(REF_OUT))
    import importlib

    return importlib.import_module("cuda_fused_sparse_splitk")


if __name__ == "__main__":
    out = build_ref(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_REFERENCE)
    print(out if out else "no reference checkout found; oracle/_ref not built")
