"""The C-ABI library loads without a GPU and exports exactly what
include/dsa_b200.h declares; the ctypes table mirrors the header."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "dsa_b200.h").read_text()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int|int64_t|const char\*)\s+(dsa_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        out[m.group(1)] = n
    return out


def test_header_declares_the_hot_path():
    names = declared_functions()
    for need in ("dsa_indexer_scan_fp8", "dsa_indexer_scan_fp8_paged", "dsa_topk_select", "dsa_sparse_mla_decode",
                 "dsa_sparse_mla_partials", "dsa_sparse_mla_combine", "dsa_quantize_e4m3_rowwise",
                 "dsa_check_device_status"):
        assert need in names


def test_library_exports_every_declared_symbol():
    from dsa_multi_layer_indexer_b200 import _lib

    handle = _lib.lib()  # raises if the library is missing or a symbol is absent
    names = declared_functions()
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)
    for name, n_args in names.items():
        assert hasattr(handle, name)
        assert len(_lib.SIGNATURES[name][1]) == n_args, name
    assert handle.dsa_abi_version() == _lib.ABI_VERSION
    m = re.search(r"#define DSA_ABI_VERSION (\d+)", HEADER)
    assert int(m.group(1)) == _lib.ABI_VERSION
    assert handle.dsa_status_string(0) == b"ok"
    assert int(handle.dsa_topk_workspace_bytes(1, 131072)) > 0


def test_bad_arguments_are_rejected_before_any_launch():
    """Argument checks run on the host: they fail the same way without a GPU."""
    from dsa_multi_layer_indexer_b200 import _lib

    h = _lib.lib()
    rc = h.dsa_sparse_mla_combine(None, None, None, None, 1, 16, 1, None)
    assert rc == -1 and b"null pointer" in h.dsa_last_error()
    buf = (ctypes.c_char * 64)()
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16
    rc = h.dsa_indexer_scan_fp8(addr, addr, addr, addr, None, addr, None, 1, 1, 24, 128, 1, 128, 128, 128, 0, None)
    assert rc == -1 and b"multiple of 16" in h.dsa_last_error()
    rc = h.dsa_topk_select(addr, None, None, None, addr, None, addr, 16, 1, 1 << 21, 1 << 21, 2048, -1, 0, None)
    assert rc == -2
    # the staging entry points: a missing operand, both cache forms missing, an unknown row format
    rc = h.dsa_indexer_stage_fp8(addr, None, addr, addr, addr, 1e-6, addr, addr, addr, addr, addr, addr, addr, None, 0, None,
                                 0, 1, 64, 128, 0, 0, 0.125, 0.088, None)
    assert rc == -1 and b"null pointer" in h.dsa_last_error()
    rc = h.dsa_indexer_stage_fp8(addr, addr, addr, addr, addr, 1e-6, addr, addr, addr, addr, addr, None, None, None, 0, None,
                                 0, 1, 64, 128, 0, 0, 0.125, 0.088, None)
    assert rc == -1 and b"dense key cache or pages" in h.dsa_last_error()
    # paged form: the page table must be able to cover every position below cap, and num_pages must be given
    rc = h.dsa_indexer_stage_fp8(addr, addr, addr, addr, addr, 1e-6, addr, addr, addr, addr, addr, None, None, addr, 4, addr,
                                 1, 1, 64, 128, 0, 0, 0.125, 0.088, None)
    assert rc == -1 and b"cannot cover" in h.dsa_last_error()
    rc = h.dsa_indexer_stage_fp8(addr, addr, addr, addr, addr, 1e-6, addr, addr, addr, addr, addr, None, None, addr, 0, addr,
                                 2, 1, 64, 128, 0, 0, 0.125, 0.088, None)
    assert rc == -1 and b"num_pages" in h.dsa_last_error()
    rc = h.dsa_latent_append(addr, addr, 1e-6, addr, addr, addr, addr, addr, 1, 128, 16, 1, 3, 0, None)
    assert rc == -1 and b"format" in h.dsa_last_error()
    # the candidate exchange: world and rank ranges, row length limit, a wait without a limit
    ptrs = (ctypes.c_void_p * 8)(*([addr] * 8))
    rc = h.dsa_topk_select_push(addr, None, None, 1, 4096, 4096, 2048, -1, 0, 9, 0, ptrs, ptrs, ptrs, addr, None)
    assert rc == -1 and b"world" in h.dsa_last_error()
    rc = h.dsa_topk_select_push(addr, None, None, 1, 4096, 4096, 2048, -1, 0, 2, 2, ptrs, ptrs, ptrs, addr, None)
    assert rc == -1 and b"rank" in h.dsa_last_error()
    rc = h.dsa_topk_select_push(addr, None, None, 1, 1 << 19, 1 << 19, 2048, -1, 0, 2, 0, ptrs, ptrs, ptrs, addr, None)
    assert rc == -2
    rc = h.dsa_topk_merge_wait(addr, addr, addr, addr, addr, 1, 2, 2048, -1, 0, None)
    assert rc == -1 and b"limit" in h.dsa_last_error()
    rc = h.dsa_ipc_open(None, 0, None)
    assert rc == -1
    # the host-integration helpers: sizes in 16-byte pieces, the one-CTA copy bounded at 1 MiB
    rc = h.dsa_copy_bytes_beside(addr, addr, 24, None)
    assert rc == -1 and b"multiples of 16" in h.dsa_last_error()
    rc = h.dsa_copy_post_epoch(addr, addr, 16, None, addr, 0, None)
    assert rc == -1 and b"null pointer" in h.dsa_last_error()
    rc = h.dsa_copy_post_epoch(addr, addr, (1 << 20) + 16, addr, addr, 1, None)
    assert rc == -1 and b"1 MiB" in h.dsa_last_error()
    # the attention that runs beside the kernel before it checks its arguments like the ordinary one
    rc = h.dsa_sparse_mla_decode_beside(addr, addr, addr, None, addr, addr, addr, addr, 1, 1, 24, 64, 1, 0.1, 128, 0, None)
    assert rc == -1 and b"multiple of 16" in h.dsa_last_error()
    rc = h.dsa_sparse_mla_decode_beside(addr, addr, addr, None, addr, addr, addr, None, 1, 1, 16, 64, 1, 0.1, 128, 0, None)
    assert rc == -1 and b"out must be" in h.dsa_last_error()


def test_staging_wrappers_reject_host_tensors():
    """The Python wrappers of the staging kernels check their operands before any launch."""
    import torch

    from dsa_multi_layer_indexer_b200 import ops

    q = torch.zeros(1, 64, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.indexer_stage_fp8(q, q[0, 0:1], torch.zeros(1, 64), torch.ones(128), torch.zeros(128), 1e-6,
                              torch.zeros(8, 32), torch.zeros(8, 32), torch.zeros(1, dtype=torch.int64),
                              torch.zeros(1, 64, 128, dtype=torch.uint8), torch.zeros(1, 64),
                              torch.zeros(1, 8, 128, dtype=torch.uint8), torch.zeros(1, 8))
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.latent_append(torch.zeros(1, 576, dtype=torch.bfloat16), torch.ones(512), 1e-6, torch.zeros(8, 32),
                          torch.zeros(8, 32), torch.zeros(1, dtype=torch.int64), torch.zeros(1, dtype=torch.int64),
                          torch.zeros(4, 656, dtype=torch.uint8))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import importlib

    from dsa_multi_layer_indexer_b200 import _lib

    monkeypatch.setenv("DSA_B200_LIB", str(tmp_path / "nope.so"))
    fresh = importlib.reload(_lib)
    try:
        with pytest.raises(ImportError):
            fresh.lib()
    finally:
        monkeypatch.delenv("DSA_B200_LIB")
        importlib.reload(_lib)


def test_default_nsplit_heuristic():
    """Host-side split heuristic: large launches of 64-head blocks get about one CTA
    per SM with a split count that divides the 64-key tiles (no empty split); small
    ones and other head counts get two 16-head CTAs per SM."""
    from dsa_multi_layer_indexer_b200 import ops

    assert ops.default_nsplit(1, 128, 2048) == 32          # 64 tiles: mma.sync kernel, 8 head blocks
    assert ops.default_nsplit(1, 16, 2048) == 32           # TP8 shape
    assert ops.default_nsplit(32, 128, 2048) == 2          # 2048 tiles: tcgen05 kernel, 64 blocks
    assert ops.default_nsplit(3, 128, 2048) == 16          # 148 // 6 = 24 -> 16 divides the 32 tiles
    for rows, heads, topk in [(2, 128, 2048), (5, 64, 1000), (8, 192, 2048), (64, 128, 512), (4, 128, 1024)]:
        n = ops.default_nsplit(rows, heads, topk)
        tiles = -(-topk // 64)
        assert 1 <= n <= tiles
        if rows * (heads // 64) * tiles >= 128:
            assert tiles % n == 0 and rows * (heads // 64) * n <= max(148, rows * (heads // 64))
