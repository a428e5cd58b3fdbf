"""ctypes binding of libdsa_b200.so (the C ABI in include/dsa_b200.h).

There is no fallback: if the library is missing or a symbol is absent the
import of this module's ``lib()`` raises, and every op in this package goes
through it. Signatures below are the single Python-side statement of the ABI;
``tests/test_abi.py`` checks them against the header.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Dict, List, Tuple

import os

_PKG = Path(__file__).resolve().parent
# DSA_B200_LIB selects another build of the same ABI (e.g. the tracing build).
LIB_PATH = Path(os.environ.get("DSA_B200_LIB") or (_PKG / "libdsa_b200.so"))

_p = C.c_void_p
_i = C.c_int
_l = C.c_int64
_f = C.c_float

# name -> (restype, argtypes)
SIGNATURES: Dict[str, Tuple[object, List[object]]] = {
    "dsa_abi_version": (_i, []),
    "dsa_last_error": (C.c_char_p, []),
    "dsa_status_string": (C.c_char_p, [_i]),
    "dsa_check_device_status": (_i, [C.POINTER(C.c_uint32)]),
    "dsa_debug_read_stamps": (_i, [_p, _i]),
    "dsa_debug_wait_timeout": (_i, [C.c_uint64, _p]),
    "dsa_indexer_scan_fp8": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _l, _l, _l, _l, _l, _i, _p]),
    "dsa_indexer_scan_fp8_paged": (_i, [_p, _p, _p, _l, _p, _l, _p, _p, _p, _i, _i, _l, _l, _p]),
    "dsa_indexer_scan_f32": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _l, _l, _l, _p]),
    "dsa_topk_workspace_bytes": (_l, [_i, _l]),
    "dsa_topk_select": (_i, [_p, _p, _p, _p, _p, _p, _p, _l, _i, _l, _l, _i, C.c_int32, C.c_int32, _p]),
    "dsa_topk_select_push": (_i, [_p, _p, _p, _i, _l, _l, _i, C.c_int32, C.c_int32, _i, _i, _p, _p, _p, _p, _p]),
    "dsa_topk_merge_wait": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, C.c_int32, _l, _p]),
    "dsa_allreduce_push": (_i, [_p, _i, _l, _i, _i, _p, _p, _p, _p]),
    "dsa_allreduce_wait_sum": (_i, [_p, _p, _p, _p, _p, _i, _l, _i, _l, _p]),
    "dsa_ipc_export": (_i, [_p, _p, _p]),
    "dsa_ipc_open": (_i, [_p, _l, _p]),
    "dsa_ipc_close": (_i, [_p, _l]),
    "dsa_topk_select_static": (_i, [_p, _p, _p, _p, _i, _l, _l, _i, C.c_int32, C.c_int32, _p]),
    "dsa_sparse_mla_partials": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _l, _i, _p]),
    "dsa_sparse_mla_combine": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "dsa_sparse_mla_decode": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _l, _i, _p]),
    "dsa_sparse_mla_decode_beside": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _l, _i, _p]),
    "dsa_fused_decode": (_i, [_p] * 15 + [_i, _i, _i, _i, _i, _f, _l, _i, _l, _l, _l, _l, _l, _p]),
    "dsa_sparse_mla_f32": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _l, _p]),
    "dsa_rmsnorm": (_i, [_p, _p, _p, _l, _i, _f, _i, _p]),
    "dsa_add_rmsnorm_bf16": (_i, [_p, _p, _p, _p, _p, _l, _i, _f, _p]),
    "dsa_silu_mul_bf16": (_i, [_p, _p, _p, _l, _p]),
    "dsa_gemv_bf16": (_i, [_p, _p, _p, _i, _i, _i, _l, _l, _p]),
    "dsa_copy_bytes": (_i, [_p, _p, _l, _p]),
    "dsa_copy_bytes_beside": (_i, [_p, _p, _l, _p]),
    "dsa_post_epoch": (_i, [_p, _p, _p]),
    "dsa_copy_post_epoch": (_i, [_p, _p, _l, _p, _p, _i, _p]),
    "dsa_indexer_stage_fp8": (_i, [_p, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _p, _p, _l, _p, _l,
                                   _i, _i, _l, _i, _i, _f, _f, _p]),
    "dsa_latent_append": (_i, [_p, _p, _f, _p, _p, _p, _p, _p, _i, _l, _l, _i, _i, _i, _p]),
    "dsa_decode_prep": (_i, [_p, _p, _p, _p, _p, _p, _l] + [_p] * 12 + [_i, _i, _i, _l, _i, _f, _p]),
    "dsa_quantize_e4m3_rowwise": (_i, [_p, _p, _p, _l, _i, _f, _p]),
}

ABI_VERSION = 9


class DsaError(RuntimeError):
    """A C-ABI call returned a negative status (the reference raises
    RuntimeError from TORCH_CHECK, kernels/cuda_fused_sparse_splitk.py:2399-2499)."""

    def __init__(self, status: int, message: str) -> None:
        super().__init__(f"dsa_b200 status {status}: {message}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built or does not match."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with "
            "`python -m dsa_multi_layer_indexer_b200.csrc.build` (there is no fallback path)"
        )
    handle = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(handle, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = res
        fn.argtypes = args
    got = handle.dsa_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {got}, this package needs {ABI_VERSION}")
    _lib = handle
    return handle


def check(status: int) -> None:
    if status != 0:
        msg = lib().dsa_last_error()
        raise DsaError(status, msg.decode("utf-8", "replace") if msg else "")


def check_device_status() -> None:
    """Synchronises and raises if any kernel's bounded wait ran out."""
    detail = C.c_uint32(0)
    check(lib().dsa_check_device_status(C.byref(detail)))
