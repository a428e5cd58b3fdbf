"""Tensor-level entry points over the C ABI: checks shapes and dtypes, hands raw
device pointers and the current CUDA stream to libdsa_b200.so.

torch is used here for device memory and streams only. Nothing in this module
computes on the host or falls back to torch kernels; a missing library raises
at the first call (``_lib.lib()``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib

LATENT_DIM = 576
VALUE_DIM = 512
INDEX_DIM = 128
HEAD_BLOCK = 16
PAGE_TOKENS = 64
INDEX_PAGE_BYTES = 8448
FP8_LATENT_ROW = 656
HIST_BINS = 4096

_FP8 = torch.float8_e4m3fn


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _cuda_contig(t: torch.Tensor, name: str, dtypes) -> None:
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.dtype in dtypes, f"{name} has dtype {t.dtype}, expected one of {dtypes}")


def _out_contig(t: torch.Tensor, name: str, dtypes) -> None:
    """An output may also live in pinned host memory (it is mapped into the device's
    address space): the kernel then writes the result straight to the host."""
    _need(t.is_cuda or t.is_pinned(), f"{name} must be a CUDA tensor or pinned host memory")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.dtype in dtypes, f"{name} has dtype {t.dtype}, expected one of {dtypes}")


def _lens(seq_lens: Optional[torch.Tensor], rows: int) -> Optional[torch.Tensor]:
    if seq_lens is not None:
        _cuda_contig(seq_lens, "seq_lens", (torch.int32,))
        _need(seq_lens.numel() == rows, f"seq_lens has {seq_lens.numel()} entries, expected {rows}")
    return seq_lens


# --------------------------------------------------------------------------- a7
def quantize_e4m3_rowwise(x: torch.Tensor, clamp_min: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row absmax e4m3 quantisation: ``(q, scale)`` with ``x ~ q * scale[..., None]``
    (reference kernels/cuda_fused_sparse_splitk.py:2969-2974)."""
    _cuda_contig(x, "x", (torch.float32,))
    cols = x.shape[-1]
    rows = x.numel() // cols
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().dsa_quantize_e4m3_rowwise(_ptr(x), _ptr(q), _ptr(scale), rows, cols,
                                                   float(clamp_min), _stream()))
    return q.view(_FP8), scale


# --------------------------------------------------------------------------- a1
def indexer_scan_fp8(
    index_q: torch.Tensor,
    index_w: torch.Tensor,
    index_k: torch.Tensor,
    k_scale: torch.Tensor,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    rows_per_seq: int = 1,
    ctx: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    hist: Optional[torch.Tensor] = None,
    impl: int = 0,
) -> torch.Tensor:
    """Indexer logits ``[R, ctx]`` (fp32) from e4m3 queries/keys.

    index_q ``[R, Hidx, 128]`` e4m3 (or uint8 bytes), index_w ``[R, Hidx]`` fp32
    with the query scale folded in, index_k ``[n_seq, cap, 128]`` (or ``[cap, 128]``),
    k_scale ``[n_seq, cap]`` fp32. Row r reads sequence ``r // rows_per_seq``.
    """
    _cuda_contig(index_q, "index_q", (_FP8, torch.uint8))
    _cuda_contig(index_w, "index_w", (torch.float32,))
    _cuda_contig(index_k, "index_k", (_FP8, torch.uint8))
    _cuda_contig(k_scale, "k_scale", (torch.float32,))
    _need(index_q.dim() == 3 and index_q.shape[-1] == INDEX_DIM, "index_q must be [R, Hidx, 128]")
    R, n_heads = index_q.shape[0], index_q.shape[1]
    _need(tuple(index_w.shape) == (R, n_heads), "index_w must be [R, Hidx]")
    if index_k.dim() == 2:
        index_k = index_k.unsqueeze(0)
        k_scale = k_scale.reshape(1, -1)
    _need(index_k.dim() == 3 and index_k.shape[-1] == INDEX_DIM, "index_k must be [n_seq, cap, 128]")
    n_seq, cap = index_k.shape[0], index_k.shape[1]
    _need(tuple(k_scale.shape) == (n_seq, cap), "k_scale must be [n_seq, cap]")
    _need(R == n_seq * rows_per_seq, f"R={R} must equal n_seq={n_seq} * rows_per_seq={rows_per_seq}")
    ctx = cap if ctx is None else int(ctx)
    _need(0 < ctx <= cap, "ctx must be in (0, cap]")
    seq_lens = _lens(seq_lens, R)
    if out is None:
        out = torch.empty(R, (ctx + 3) // 4 * 4, dtype=torch.float32, device=index_q.device)
    _cuda_contig(out, "out", (torch.float32,))
    _need(out.dim() == 2 and out.shape[0] == R and out.shape[1] >= ctx, "out must be [R, >= ctx]")
    if hist is not None:
        _cuda_contig(hist, "hist", (torch.int32, torch.uint32))
        _need(hist.numel() == R * HIST_BINS, "hist must be [R, 4096]")
    _lib.check(_lib.lib().dsa_indexer_scan_fp8(
        _ptr(index_q), _ptr(index_w), _ptr(index_k), _ptr(k_scale), _ptr(seq_lens), _ptr(out),
        _ptr(hist), R, rows_per_seq, n_heads, ctx, n_seq, cap, cap, out.shape[1], impl, _stream()))
    return out[:, :ctx]


def indexer_scan_fp8_paged(
    index_q: torch.Tensor,
    index_w: torch.Tensor,
    index_k_pages: torch.Tensor,
    page_table: torch.Tensor,
    seq_lens: torch.Tensor,
    ctx: int,
    *,
    out: Optional[torch.Tensor] = None,
    hist: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Paged form: index_k_pages ``[num_pages, 8448]`` uint8, page_table ``[R, pt_stride]`` int32."""
    _cuda_contig(index_q, "index_q", (_FP8, torch.uint8))
    _cuda_contig(index_w, "index_w", (torch.float32,))
    _cuda_contig(index_k_pages, "index_k_pages", (torch.uint8,))
    _cuda_contig(page_table, "page_table", (torch.int32,))
    _need(index_q.dim() == 3 and index_q.shape[-1] == INDEX_DIM, "index_q must be [R, Hidx, 128]")
    R, n_heads = index_q.shape[0], index_q.shape[1]
    _need(index_k_pages.dim() == 2 and index_k_pages.shape[1] == INDEX_PAGE_BYTES,
          "index_k_pages must be [num_pages, 8448]")
    _need(page_table.dim() == 2 and page_table.shape[0] == R, "page_table must be [R, pt_stride]")
    seq_lens = _lens(seq_lens, R)
    _need(seq_lens is not None, "paged scan needs seq_lens")
    if out is None:
        out = torch.empty(R, (ctx + 3) // 4 * 4, dtype=torch.float32, device=index_q.device)
    _cuda_contig(out, "out", (torch.float32,))
    _need(out.dim() == 2 and out.shape[0] == R and out.shape[1] >= ctx, "out must be [R, >= ctx]")
    _need(tuple(index_w.shape) == (R, n_heads), "index_w must be [R, Hidx]")
    _need(page_table.shape[1] * PAGE_TOKENS >= ctx, "page_table rows cannot cover ctx positions")
    if hist is not None:
        _cuda_contig(hist, "hist", (torch.int32, torch.uint32))
        _need(hist.numel() == R * HIST_BINS, "hist must be [R, 4096]")
    _lib.check(_lib.lib().dsa_indexer_scan_fp8_paged(
        _ptr(index_q), _ptr(index_w), _ptr(index_k_pages), index_k_pages.shape[0], _ptr(page_table),
        page_table.shape[1], _ptr(seq_lens), _ptr(out), _ptr(hist), R, n_heads, int(ctx),
        out.shape[1], _stream()))
    return out[:, :ctx]


def indexer_scan_f32(
    index_q: torch.Tensor,
    index_w: torch.Tensor,
    index_k: torch.Tensor,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    rows_per_seq: int = 1,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """fp32 logits for any head count / key width: q ``[R, H, D]``, k ``[n_seq, ctx, D]``."""
    for t, n in ((index_q, "index_q"), (index_w, "index_w"), (index_k, "index_k")):
        _cuda_contig(t, n, (torch.float32,))
    R, n_heads, d = index_q.shape
    if index_k.dim() == 2:
        index_k = index_k.unsqueeze(0)
    n_seq, ctx = index_k.shape[0], index_k.shape[1]
    _need(index_k.shape[2] == d, "index_k width differs from index_q")
    _need(R == n_seq * rows_per_seq, "R must equal n_seq * rows_per_seq")
    seq_lens = _lens(seq_lens, R)
    if out is None:
        out = torch.empty(R, (ctx + 3) // 4 * 4, dtype=torch.float32, device=index_q.device)
    _lib.check(_lib.lib().dsa_indexer_scan_f32(
        _ptr(index_q), _ptr(index_w), _ptr(index_k), _ptr(seq_lens), _ptr(out), R, rows_per_seq,
        n_heads, d, ctx, ctx, out.shape[1], _stream()))
    return out[:, :ctx]


# --------------------------------------------------------------------------- a3
def topk_workspace(rows: int, n: int, device) -> torch.Tensor:
    """Zeroed scratch for ``topk_select`` on ``rows`` rows of ``n`` logits. It is
    left re-armed by every call, so one allocation serves a whole decode loop;
    calls that share it must not overlap on the device."""
    nbytes = int(_lib.lib().dsa_topk_workspace_bytes(rows, n))
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def topk_select(
    logits: torch.Tensor,
    topk: int,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    hist: Optional[torch.Tensor] = None,
    index_map: Optional[torch.Tensor] = None,
    pad_value: int = -1,
    index_offset: int = 0,
    out_idx: Optional[torch.Tensor] = None,
    out_val: Optional[torch.Tensor] = None,
    return_values: bool = False,
    workspace: Optional[torch.Tensor] = None,
):
    """Exact top-k per row of ``logits[R, n]`` (a view of a wider slab is fine):
    int32 positions in ascending order, ties to the lower position, padded with
    ``pad_value``."""
    _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2, "logits must be CUDA fp32 [R, n]")
    _need(logits.stride(1) == 1, "logits rows must be dense")
    R, n = logits.shape
    slab_stride = logits.stride(0) if R > 1 else max(logits.stride(0), n)
    seq_lens = _lens(seq_lens, R)
    if index_map is not None:
        _cuda_contig(index_map, "index_map", (torch.int32,))
        _need(tuple(index_map.shape) == (R, n), "index_map must be [R, n]")
    if out_idx is None:
        out_idx = torch.empty(R, topk, dtype=torch.int32, device=logits.device)
    _cuda_contig(out_idx, "out_idx", (torch.int32,))
    _need(tuple(out_idx.shape) == (R, topk), f"out_idx must be [R, topk] = [{R}, {topk}]")
    if out_val is None and return_values:
        out_val = torch.empty(R, topk, dtype=torch.float32, device=logits.device)
    if out_val is not None:
        _cuda_contig(out_val, "out_val", (torch.float32,))
        _need(tuple(out_val.shape) == (R, topk), f"out_val must be [R, topk] = [{R}, {topk}]")
    if hist is not None:
        _cuda_contig(hist, "hist", (torch.int32, torch.uint32))
        _need(hist.numel() == R * HIST_BINS, "hist must be [R, 4096]")
    if workspace is None:
        # a fresh zeroed scratch per call is always safe; steady-state callers pass their own
        workspace = topk_workspace(R, n, logits.device)
    _cuda_contig(workspace, "workspace", (torch.uint8,))
    _need(0 < int(topk) <= 65536, "topk must be in [1, 65536]")
    _lib.check(_lib.lib().dsa_topk_select(
        _ptr(logits), _ptr(seq_lens), _ptr(hist), _ptr(index_map), _ptr(out_idx), _ptr(out_val),
        _ptr(workspace), workspace.numel(), R, n, slab_stride, int(topk), int(pad_value),
        int(index_offset), _stream()))
    if return_values or out_val is not None:
        return out_idx, out_val
    return out_idx


# --------------------------------------------------------------------------- a4, a5
class MlaScratch:
    """Caller-owned split-K partials (the reference's PartAcc / PartM / PartL,
    kernels/cuda_fused_sparse_splitk.py:3005-3009), sized once and reused."""

    def __init__(self, rows: int, heads: int, nsplit: int, device) -> None:
        self.rows, self.heads, self.nsplit = rows, heads, nsplit
        self.acc = torch.empty(rows, nsplit, heads, VALUE_DIM, dtype=torch.float32, device=device)
        self.m = torch.empty(rows, nsplit, heads, dtype=torch.float32, device=device)
        self.l = torch.empty(rows, nsplit, heads, dtype=torch.float32, device=device)


def default_nsplit(rows: int, heads: int, topk: int, sm_count: int = 148) -> int:
    """Splits of the index list, each a whole number of 64-key tiles. Head counts
    that are a multiple of 64 run on the tcgen05 kernel (one CTA per SM, 64 heads
    per CTA) once the launch has 128 tiles of 64 heads x 64 keys: about one CTA per
    SM in total, and a split count that divides the tiles so no split is empty.
    Smaller launches and other head counts run on the mma.sync kernel (16 heads
    per CTA, two CTAs per SM)."""
    tiles = max(1, math.ceil(topk / 64))
    if heads % 64 == 0 and rows * (heads // 64) * tiles >= 128:
        blocks = max(1, rows * (heads // 64))
        want = max(1, min(sm_count // blocks, tiles))
        while tiles % want:
            want -= 1
        return want
    blocks = max(1, rows * (heads // HEAD_BLOCK))
    want = max(1, (2 * sm_count) // blocks)
    return max(1, min(want, tiles))


def sparse_mla_decode(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: Optional[torch.Tensor],
    sm_scale: float,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    rows_per_seq: int = 1,
    nsplit: Optional[int] = None,
    scratch: Optional[MlaScratch] = None,
    out: Optional[torch.Tensor] = None,
    dense_keys: Optional[int] = None,
    stage: str = "both",
    beside_previous: bool = False,
) -> torch.Tensor:
    """Sparse MLA decode: q ``[R, H, 576]`` bf16, kv ``[n_seq, cap, 576]`` bf16 or
    ``[n_seq, cap, 656]`` uint8 (fp8-packed rows), indices ``[R, topk]`` int32 or
    None for dense attention over ``dense_keys`` positions. Returns ``[R, H, 512]`` bf16.
    ``beside_previous``: none of the operands comes from the two kernels enqueued just before
    this call (the lagged schedule's attention behind this layer's scan and top-k); the attention
    then runs beside the top-k and completes after it."""
    _cuda_contig(q, "q", (torch.bfloat16,))
    _need(q.dim() == 3 and q.shape[2] == LATENT_DIM, "q must be [R, H, 576]")
    R, H = q.shape[0], q.shape[1]
    _need(H % HEAD_BLOCK == 0, f"H={H} must be a multiple of {HEAD_BLOCK} (pad heads with zero queries)")
    if kv.dim() == 2:
        kv = kv.unsqueeze(0)
    _need(kv.is_cuda and kv.is_contiguous() and kv.dim() == 3, "kv must be a contiguous CUDA [n_seq, cap, w] tensor")
    if kv.dtype == torch.bfloat16:
        _need(kv.shape[2] == LATENT_DIM, "bf16 kv rows must be 576 wide")
        kv_fp8 = 0
    else:
        _need(kv.dtype == torch.uint8 and kv.shape[2] == FP8_LATENT_ROW, "fp8 kv rows must be 656 bytes of uint8")
        kv_fp8 = 1
    n_seq, cap = kv.shape[0], kv.shape[1]
    _need(R == n_seq * rows_per_seq, "R must equal n_seq * rows_per_seq")
    if indices is not None:
        _cuda_contig(indices, "indices", (torch.int32,))
        _need(indices.dim() == 2 and indices.shape[0] == R, "indices must be [R, topk]")
        topk = indices.shape[1]
    else:
        topk = int(dense_keys if dense_keys is not None else cap)
    seq_lens = _lens(seq_lens, R)
    if nsplit is None:
        nsplit = scratch.nsplit if scratch is not None else default_nsplit(R, H, topk)
    if scratch is None:
        scratch = MlaScratch(R, H, nsplit, q.device)
    _need(scratch.rows >= R and scratch.heads == H and scratch.nsplit == nsplit, "scratch does not match the launch")
    if out is None:
        out = torch.empty(R, H, VALUE_DIM, dtype=torch.bfloat16, device=q.device)
    _out_contig(out, "out", (torch.bfloat16,))
    _need(not beside_previous or stage == "both", "beside_previous goes with stage='both'")
    if stage == "both":
        fn = _lib.lib().dsa_sparse_mla_decode_beside if beside_previous else _lib.lib().dsa_sparse_mla_decode
        _lib.check(fn(
            _ptr(q), _ptr(kv), _ptr(indices), _ptr(seq_lens), _ptr(scratch.acc), _ptr(scratch.m),
            _ptr(scratch.l), _ptr(out), R, rows_per_seq, H, topk, nsplit, float(sm_scale), cap, kv_fp8,
            _stream()))
    elif stage == "partials":  # the two halves separately, as the reference schedules them
        _lib.check(_lib.lib().dsa_sparse_mla_partials(
            _ptr(q), _ptr(kv), _ptr(indices), _ptr(seq_lens), _ptr(scratch.acc), _ptr(scratch.m),
            _ptr(scratch.l), R, rows_per_seq, H, topk, nsplit, float(sm_scale), cap, kv_fp8, _stream()))
    elif stage == "combine":
        _lib.check(_lib.lib().dsa_sparse_mla_combine(
            _ptr(scratch.acc), _ptr(scratch.m), _ptr(scratch.l), _ptr(out), R, H, nsplit, _stream()))
    else:
        raise ValueError(f"unknown stage {stage!r}")
    return out


def sparse_mla_f32(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: Optional[torch.Tensor],
    value_dim: int,
    sm_scale: float,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    rows_per_seq: int = 1,
) -> torch.Tensor:
    """fp32 attention for any width: q ``[R, H, Dqk]``, kv ``[n_seq, ctx, Dqk]``;
    indices None = dense causal over ``seq_lens``."""
    _cuda_contig(q, "q", (torch.float32,))
    _cuda_contig(kv, "kv", (torch.float32,))
    if kv.dim() == 2:
        kv = kv.unsqueeze(0)
    R, H, dqk = q.shape
    n_seq, ctx = kv.shape[0], kv.shape[1]
    _need(kv.shape[2] == dqk and R == n_seq * rows_per_seq, "q / kv shapes disagree")
    topk = 0
    if indices is not None:
        _cuda_contig(indices, "indices", (torch.int32,))
        topk = indices.shape[1]
    seq_lens = _lens(seq_lens, R)
    out = torch.empty(R, H, value_dim, dtype=torch.float32, device=q.device)
    _lib.check(_lib.lib().dsa_sparse_mla_f32(
        _ptr(q), _ptr(kv), _ptr(indices), _ptr(seq_lens), _ptr(out), R, rows_per_seq, H, dqk,
        value_dim, topk, float(sm_scale), ctx, _stream()))
    return out


# --------------------------------------------------------------------------- a6
def fused_decode(
    q: torch.Tensor,
    kv: torch.Tensor,
    attend_indices: torch.Tensor,
    sm_scale: float,
    index_q: torch.Tensor,
    index_w: torch.Tensor,
    index_k: torch.Tensor,
    k_scale: torch.Tensor,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    rows_per_seq: int = 1,
    nsplit: Optional[int] = None,
    scratch: Optional[MlaScratch] = None,
    out: Optional[torch.Tensor] = None,
    logits: Optional[torch.Tensor] = None,
    hist: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """One launch for a layer's sparse MLA over ``attend_indices`` AND its indexer
    scan (then the LSE merge): returns ``(attention_out [R,H,512] bf16, logits [R,ctx] fp32)``.
    Same operands as :func:`sparse_mla_decode` (bf16 cache) and :func:`indexer_scan_fp8`."""
    _cuda_contig(q, "q", (torch.bfloat16,))
    _need(q.dim() == 3 and q.shape[2] == LATENT_DIM and q.shape[1] % HEAD_BLOCK == 0, "q must be [R, H % 16 == 0, 576]")
    R, H = q.shape[0], q.shape[1]
    if kv.dim() == 2:
        kv = kv.unsqueeze(0)
    _cuda_contig(kv, "kv", (torch.bfloat16,))
    _need(kv.dim() == 3 and kv.shape[2] == LATENT_DIM, "kv must be [n_seq, cap, 576] bf16")
    _cuda_contig(attend_indices, "attend_indices", (torch.int32,))
    _need(attend_indices.dim() == 2 and attend_indices.shape[0] == R, "attend_indices must be [R, topk]")
    topk = attend_indices.shape[1]
    _cuda_contig(index_q, "index_q", (_FP8, torch.uint8))
    _cuda_contig(index_w, "index_w", (torch.float32,))
    _cuda_contig(index_k, "index_k", (_FP8, torch.uint8))
    _cuda_contig(k_scale, "k_scale", (torch.float32,))
    if index_k.dim() == 2:
        index_k = index_k.unsqueeze(0)
        k_scale = k_scale.reshape(1, -1)
    n_seq, cap = index_k.shape[0], index_k.shape[1]
    _need(kv.shape[0] == n_seq and R == n_seq * rows_per_seq, "R must equal n_seq * rows_per_seq for both caches")
    _need(index_q.shape[0] == R and tuple(index_w.shape) == (R, index_q.shape[1]), "index_q / index_w rows differ from q")
    seq_lens = _lens(seq_lens, R)
    if nsplit is None:
        nsplit = scratch.nsplit if scratch is not None else default_nsplit(R, H, topk)
    if scratch is None:
        scratch = MlaScratch(R, H, nsplit, q.device)
    _need(scratch.rows >= R and scratch.heads == H and scratch.nsplit == nsplit, "scratch does not match the launch")
    if out is None:
        out = torch.empty(R, H, VALUE_DIM, dtype=torch.bfloat16, device=q.device)
    if logits is None:
        logits = torch.empty(R, (cap + 3) // 4 * 4, dtype=torch.float32, device=q.device)
    _cuda_contig(logits, "logits", (torch.float32,))
    if hist is not None:
        _cuda_contig(hist, "hist", (torch.int32, torch.uint32))
        _need(hist.numel() == R * HIST_BINS, "hist must be [R, 4096]")
    _lib.check(_lib.lib().dsa_fused_decode(
        _ptr(q), _ptr(kv), _ptr(attend_indices), _ptr(seq_lens), _ptr(scratch.acc), _ptr(scratch.m),
        _ptr(scratch.l), _ptr(out), _ptr(index_q), _ptr(index_w), _ptr(index_k), _ptr(k_scale), _ptr(seq_lens),
        _ptr(logits), _ptr(hist), R, rows_per_seq, H, topk, nsplit, float(sm_scale), kv.shape[1],
        index_q.shape[1], cap, n_seq, cap, cap, logits.shape[1], _stream()))
    return out, logits[:, :cap]


# --------------------------------------------------------------------------- decode-step preparation
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last dimension in one launch (fp32 math, one rounding)."""
    _need(x.is_cuda and x.dtype in (torch.float32, torch.bfloat16), "x must be CUDA fp32 / bf16")
    x = x.contiguous()
    w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    out = torch.empty_like(x)
    dim = x.shape[-1]
    _lib.check(_lib.lib().dsa_rmsnorm(_ptr(x), _ptr(w.contiguous()), _ptr(out), x.numel() // dim, dim, float(eps),
                                      0 if x.dtype == torch.float32 else 1, _stream()))
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float):
    """``s = x + delta`` and ``rmsnorm(s)`` in one launch (bf16 rows of at most 8192
    elements, a multiple of 8): returns ``(s, normed)``, both rounded exactly as the
    separate addition and norm would be."""
    _need(x.is_cuda and x.dtype == torch.bfloat16 and delta.dtype == torch.bfloat16 and x.shape == delta.shape,
          "x and delta must be CUDA bf16 tensors of one shape")
    dim = x.shape[-1]
    _need(dim % 8 == 0 and dim <= 8192, "the row length must be a multiple of 8 and at most 8192")
    x, delta = x.contiguous(), delta.contiguous()
    w = (weight if weight.dtype == x.dtype else weight.to(x.dtype)).contiguous()
    s, out = torch.empty_like(x), torch.empty_like(x)
    _lib.check(_lib.lib().dsa_add_rmsnorm_bf16(_ptr(x), _ptr(delta), _ptr(w), _ptr(s), _ptr(out), x.numel() // dim, dim,
                                               float(eps), _stream()))
    return s, out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` over bf16 tensors in one launch, rounded as the two separate operations."""
    _need(gate.is_cuda and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.shape == up.shape,
          "gate and up must be CUDA bf16 tensors of one shape")
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(gate)
    _lib.check(_lib.lib().dsa_silu_mul_bf16(_ptr(gate), _ptr(up), _ptr(out), gate.numel(), _stream()))
    return out


def copy_bytes(dst: torch.Tensor, src: torch.Tensor, beside_previous: bool = False) -> None:
    """``dst <- src`` (same byte count, a multiple of 16) by a kernel on the current stream.
    Each side is a contiguous CUDA tensor or pinned host memory. With ``beside_previous`` the
    copy runs beside the kernel enqueued just before it and completes after it; what is enqueued
    next sees both. Neither of the two kernels enqueued before it may write or read these bytes
    (the top-k releases its dependents before it waits for the scan)."""
    for t, name in ((dst, "dst"), (src, "src")):
        _need((t.is_cuda or t.is_pinned()) and t.is_contiguous(), f"{name} must be contiguous CUDA or pinned memory")
    nbytes = dst.numel() * dst.element_size()
    _need(nbytes == src.numel() * src.element_size() and nbytes % 16 == 0, "byte counts must match and be a multiple of 16")
    fn = _lib.lib().dsa_copy_bytes_beside if beside_previous else _lib.lib().dsa_copy_bytes
    _lib.check(fn(_ptr(dst), _ptr(src), nbytes, _stream()))


def post_epoch(counter: torch.Tensor, host_flag: torch.Tensor) -> None:
    """Enqueues the completion signal: ``counter`` (one int32 on the device) is bumped and
    its value posted to ``host_flag`` (one int32 of pinned host memory) after everything
    enqueued so far on the current stream."""
    _need(counter.is_cuda and counter.dtype == torch.int32 and counter.numel() == 1, "counter: one CUDA int32")
    _need(host_flag.is_pinned() and host_flag.dtype == torch.int32 and host_flag.numel() == 1,
          "host_flag: one pinned int32")
    _lib.check(_lib.lib().dsa_post_epoch(_ptr(counter), _ptr(host_flag), _stream()))


def copy_post_epoch(dst: torch.Tensor, src: torch.Tensor, counter: torch.Tensor, host_flag: torch.Tensor,
                    beside_previous: bool = False) -> None:
    """:func:`copy_bytes` of at most 1 MiB followed by :func:`post_epoch`, as one launch: the last
    node of a step when a few KB (the selection) still have to reach the host before the signal.
    ``beside_previous``: ``src`` does not come from the two kernels enqueued before this call; it is
    copied beside the last of them and only the signal waits for it."""
    for t, name in ((dst, "dst"), (src, "src")):
        _need((t.is_cuda or t.is_pinned()) and t.is_contiguous(), f"{name} must be contiguous CUDA or pinned memory")
    nbytes = dst.numel() * dst.element_size()
    _need(nbytes == src.numel() * src.element_size() and nbytes % 16 == 0 and nbytes <= 1 << 20,
          "byte counts must match, be a multiple of 16 and at most 1 MiB")
    _need(counter.is_cuda and counter.dtype == torch.int32 and counter.numel() == 1, "counter: one CUDA int32")
    _need(host_flag.is_pinned() and host_flag.dtype == torch.int32 and host_flag.numel() == 1,
          "host_flag: one pinned int32")
    _lib.check(_lib.lib().dsa_copy_post_epoch(_ptr(dst), _ptr(src), nbytes, _ptr(counter), _ptr(host_flag),
                                              1 if beside_previous else 0, _stream()))


def gemv(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` for a decode batch of 1..4 rows (bf16, fp32 accumulation): the weight
    matrix ``[n, k]`` is streamed once. For the projection shapes where the library GEMV is
    latency-bound."""
    _need(x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2,
          "x must be a CUDA bf16 [B, k] tensor and weight bf16")
    b, k = x.shape
    n = weight.shape[0]
    _need(weight.dim() == 2 and weight.shape[1] == k and weight.is_contiguous(), "weight must be contiguous [n, k]")
    _need(1 <= b <= 4 and k % 8 == 0 and b * k * 2 <= 96 * 1024, "batch 1..4, k a multiple of 8, batch * k <= 48K")
    x = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 else x.contiguous()
    y = torch.empty(b, n, dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.lib().dsa_gemv_bf16(_ptr(weight), _ptr(x), _ptr(y), b, n, k, x.stride(0) if b > 1 else k, n,
                                        _stream()))
    return y


def indexer_stage_fp8(q_raw, k_raw, w_raw, k_norm_weight, k_norm_bias, k_norm_eps: float, rope_cos, rope_sin,
                      positions, index_q, index_w, cache_index_k=None, cache_k_scale=None, pages=None,
                      page_table=None, rope_interleave: bool = False, scale_fmt: Optional[str] = None,
                      softmax_scale: Optional[float] = None) -> None:
    """Serving-form indexer staging in one launch: the reference's
    ``Indexer.stage_fp8_operands`` after its three projections
    (inference/modeling/transformer.py:1015-1066) -- LayerNorm of the key, rotary
    embedding, Hadamard rotation, ``act_quant`` (``scale_fmt`` not None = power-of-two
    scales), folded head weights, and the append of the key to the dense cache
    (``cache_index_k`` [B, cap, 128] u8 + ``cache_k_scale`` [B, cap]) or to 64-token
    ``pages`` through ``page_table``. ``q_raw`` [B, heads, 128] / ``k_raw`` [B, 128] bf16,
    ``w_raw`` [B, heads] fp32, ``rope_cos`` / ``rope_sin`` [cap, 32] fp32."""
    _cuda_contig(q_raw, "q_raw", (torch.bfloat16,))
    _cuda_contig(k_raw, "k_raw", (torch.bfloat16,))
    for t, n in ((w_raw, "w_raw"), (k_norm_weight, "k_norm_weight"), (k_norm_bias, "k_norm_bias"),
                 (rope_cos, "rope_cos"), (rope_sin, "rope_sin"), (index_w, "index_w")):
        _cuda_contig(t, n, (torch.float32,))
    _cuda_contig(positions, "positions", (torch.int64,))
    _cuda_contig(index_q, "index_q", (torch.uint8, torch.float8_e4m3fn))
    _need(q_raw.dim() == 3 and q_raw.shape[2] == INDEX_DIM, "q_raw must be [B, heads, 128]")
    B, n_heads = q_raw.shape[0], q_raw.shape[1]
    _need(k_raw.shape == (B, INDEX_DIM) and w_raw.shape == (B, n_heads) and index_w.shape == (B, n_heads)
          and index_q.shape == q_raw.shape and positions.shape == (B,), "operand shapes disagree")
    _need(k_norm_weight.numel() == INDEX_DIM and k_norm_bias.numel() == INDEX_DIM, "LayerNorm parameters must be [128]")
    cap = rope_cos.shape[0]
    _need(rope_cos.shape == (cap, 32) and rope_sin.shape == (cap, 32), "rotary tables must be [cap, 32]")
    paged = pages is not None
    if paged:
        _cuda_contig(pages, "pages", (torch.uint8,))
        _cuda_contig(page_table, "page_table", (torch.int32,))
        _need(page_table.dim() == 2 and page_table.shape[0] == B, "page_table must be [B, pages per sequence]")
        _need(pages.numel() % INDEX_PAGE_BYTES == 0, "page pool must be whole pages")
        cap = min(cap, page_table.shape[1] * PAGE_TOKENS)
    else:
        _cuda_contig(cache_index_k, "cache_index_k", (torch.uint8, torch.float8_e4m3fn))
        _cuda_contig(cache_k_scale, "cache_k_scale", (torch.float32,))
        _need(cache_index_k.dim() == 3 and cache_index_k.shape[0] == B and cache_index_k.shape[2] == INDEX_DIM
              and cache_k_scale.shape == cache_index_k.shape[:2], "caches must be [B, cap, 128] and [B, cap]")
        cap = min(cap, cache_index_k.shape[1])
    if softmax_scale is None:
        softmax_scale = INDEX_DIM ** -0.5
    _lib.check(_lib.lib().dsa_indexer_stage_fp8(
        _ptr(q_raw), _ptr(k_raw), _ptr(w_raw), _ptr(k_norm_weight), _ptr(k_norm_bias), float(k_norm_eps),
        _ptr(rope_cos), _ptr(rope_sin), _ptr(positions), _ptr(index_q), _ptr(index_w),
        _ptr(cache_index_k) if not paged else None, _ptr(cache_k_scale) if not paged else None,
        _ptr(pages) if paged else None, pages.numel() // INDEX_PAGE_BYTES if paged else 0,
        _ptr(page_table) if paged else None, page_table.shape[1] if paged else 0, B, n_heads, cap, 1 if rope_interleave else 0,
        0 if scale_fmt is None else 1, float(n_heads ** -0.5), float(softmax_scale), _stream()))


def latent_append(kv_a, kv_norm_weight, eps: float, rope_cos, rope_sin, positions, slots, pool,
                  rope_interleave: bool = True, fmt: str = "fp8", scale_fmt: Optional[str] = None) -> None:
    """Serving-form latent append in one launch (inference/modeling/transformer.py:3264-3276
    in the reference): RMSNorm of the 512 latent dims of ``kv_a`` [B, 576] bf16, rotary
    embedding of its 64 rope dims, row written at ``slots[b]`` of ``pool``: ``fmt="bf16"``
    [n_slots, 576] bf16 as it is, ``"bf16_quant"`` the same with the latent dims passed
    through act_quant and back, ``"fp8"`` the 656-byte packed rows [n_slots, 656] uint8."""
    _cuda_contig(kv_a, "kv_a", (torch.bfloat16,))
    for t, n in ((kv_norm_weight, "kv_norm_weight"), (rope_cos, "rope_cos"), (rope_sin, "rope_sin")):
        _cuda_contig(t, n, (torch.float32,))
    _cuda_contig(positions, "positions", (torch.int64,))
    _cuda_contig(slots, "slots", (torch.int64,))
    _need(kv_a.dim() == 2 and kv_a.shape[1] == LATENT_DIM, "kv_a must be [B, 576]")
    B = kv_a.shape[0]
    _need(positions.shape == (B,) and slots.shape == (B,), "positions and slots must be [B]")
    _need(kv_norm_weight.numel() == VALUE_DIM, "kv_norm_weight must be [512]")
    cap = rope_cos.shape[0]
    _need(rope_cos.shape == (cap, 32) and rope_sin.shape == (cap, 32), "rotary tables must be [cap, 32]")
    formats = {"bf16": 0, "bf16_quant": 1, "fp8": 2}
    _need(fmt in formats, f"fmt must be one of {sorted(formats)}")
    if fmt == "fp8":
        _cuda_contig(pool, "pool", (torch.uint8,))
        _need(pool.dim() == 2 and pool.shape[1] == FP8_LATENT_ROW, "an fp8 pool is [n_slots, 656] uint8")
    else:
        _cuda_contig(pool, "pool", (torch.bfloat16,))
        _need(pool.dim() == 2 and pool.shape[1] == LATENT_DIM, "a bf16 pool is [n_slots, 576]")
    _lib.check(_lib.lib().dsa_latent_append(
        _ptr(kv_a), _ptr(kv_norm_weight), float(eps), _ptr(rope_cos), _ptr(rope_sin), _ptr(positions), _ptr(slots),
        _ptr(pool), B, cap, pool.shape[0], 1 if rope_interleave else 0, formats[fmt],
        0 if scale_fmt is None else 1, _stream()))


def decode_prep(iq_raw, w_raw, ik_raw, kv_a, q_abs, q_pe, kv_norm_w, mla_cos, mla_sin, idx_cos, idx_sin,
                positions, index_q, index_w, q_full, cache_index_k, cache_k_scale, cache_kv,
                interleave: bool, eps: float) -> None:
    """One launch for the chain between the projection GEMVs and the hot path
    (see ``dsa_decode_prep`` in the header). All operands bf16 CUDA tensors;
    ``q_pe`` may be a strided view ``q[..., nope:]`` of the q_b_proj output."""
    for t, n in ((iq_raw, "iq_raw"), (w_raw, "w_raw"), (ik_raw, "ik_raw"), (kv_a, "kv_a"), (q_abs, "q_abs"),
                 (kv_norm_w, "kv_norm_w"), (mla_cos, "mla_cos"), (mla_sin, "mla_sin"), (idx_cos, "idx_cos"),
                 (idx_sin, "idx_sin")):
        _cuda_contig(t, n, (torch.bfloat16,))
    _need(q_pe.dtype == torch.bfloat16 and q_pe.dim() == 3 and q_pe.shape[2] == 64 and q_pe.stride(2) == 1
          and (q_pe.shape[0] == 1 or q_pe.stride(0) == q_pe.shape[1] * q_pe.stride(1)),
          "q_pe must be a [B, H, 64] bf16 view with dense rows")
    _cuda_contig(positions, "positions", (torch.int64,))
    B, n_idx = iq_raw.shape[0], iq_raw.shape[1]
    H = q_abs.shape[1]
    _need(iq_raw.shape[2] == INDEX_DIM and kv_a.shape[-1] == LATENT_DIM and q_abs.shape[2] == VALUE_DIM,
          "decode prep needs the production geometry")
    cap = cache_kv.shape[1]
    _need(cache_kv.shape[0] == B and cache_index_k.shape[:2] == (B, cap), "caches must be [B, cap, ...]")
    _lib.check(_lib.lib().dsa_decode_prep(
        _ptr(iq_raw), _ptr(w_raw), _ptr(ik_raw), _ptr(kv_a), _ptr(q_abs), _ptr(q_pe), q_pe.stride(1), _ptr(kv_norm_w),
        _ptr(mla_cos), _ptr(mla_sin), _ptr(idx_cos), _ptr(idx_sin), _ptr(positions), _ptr(index_q), _ptr(index_w),
        _ptr(q_full), _ptr(cache_index_k), _ptr(cache_k_scale), _ptr(cache_kv), B, H, n_idx, cap,
        1 if interleave else 0, float(eps), _stream()))


# --------------------------------------------------------------------------- exchanges between GPUs
class PeerArena:
    """ONE zeroed device allocation per rank that the other ranks of a node store into, plus the
    addresses under which this process reaches every rank's copy. Those come from CUDA IPC
    (``connect``: one process per GPU, handles exchanged over the process group) or, for ranks
    emulated on one GPU, are simply the other objects' own pointers (``local_group``)."""

    def __init__(self, nbytes: int, world: int, rank: int, device) -> None:
        import ctypes as C

        _need(1 <= world <= 8 and 0 <= rank < world, "world must be 1..8 and rank inside it")
        self.world, self.rank = world, rank
        self.arena = torch.zeros((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=device)
        self._bases = [None] * world       # every rank's arena as this process addresses it
        self._bases[rank] = self.arena.data_ptr()
        self._opened = []                  # (mapped pointer, offset) of the peers' allocations
        self._C = C

    def _peer_pointers(self, offset: int):
        """ctypes array of ``world`` pointers: byte ``offset`` of every rank's arena."""
        _need(all(b is not None for b in self._bases), "not every rank's buffer is mapped: call connect() first")
        return (self._C.c_void_p * self.world)(*[b + offset for b in self._bases])

    def _mapped(self) -> None:
        """Hook: called once every rank's arena is addressable."""

    def connect(self, group=None):
        """One process per GPU: exchanges CUDA IPC handles of the arenas over ``group`` and maps
        the peers' arenas. Collective: every rank of the group calls it."""
        import torch.distributed as dist

        C = self._C
        if self.world > 1:
            handle = (C.c_ubyte * 64)()
            offset = C.c_int64(0)
            _lib.check(_lib.lib().dsa_ipc_export(self.arena.data_ptr(), handle, C.byref(offset)))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, (bytes(handle), int(offset.value)), group=group)
            for r, (h, off) in enumerate(everyone):
                if r == self.rank:
                    continue
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                out = C.c_void_p(0)
                _lib.check(_lib.lib().dsa_ipc_open(buf, off, C.byref(out)))
                self._bases[r] = int(out.value)
                self._opened.append((int(out.value), off))
        self._mapped()
        if self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=group)  # nobody stores before every arena is zeroed and mapped
        return self

    @classmethod
    def local_group(cls, *args, world: int, **kwargs):
        """``world`` ranks emulated on ONE GPU (tests, single-GPU checks): every "peer" buffer is
        an ordinary local allocation. The ranks' launches must then be enqueued one after the
        other on one stream, every push before the first wait."""
        xs = [cls(*args, world=world, rank=r, **kwargs) for r in range(world)]
        for x in xs:
            x._bases = [y.arena.data_ptr() for y in xs]
            x._mapped()
        return xs

    def close(self) -> None:
        for ptr, off in self._opened:
            _lib.lib().dsa_ipc_close(ptr, off)
        self._opened = []


class CandidateExchange(PeerArena):
    """One rank's side of the candidate exchange of a KV-sequence-sharded indexer
    (``dsa_topk_select_push`` / ``dsa_topk_merge_wait``): this rank's gather buffers
    ``[2, rows, world, topk]`` (index and logit), the flag words the other ranks post to and
    the two step counters. After set-up a step is two launches and touches no host state."""

    def __init__(self, rows: int, topk: int, world: int, rank: int, device, wait_limit_s: float = 2.0) -> None:
        self.rows, self.topk = rows, topk
        self.wait_limit_ns = int(wait_limit_s * 1e9)
        n_gather = 2 * rows * world * topk
        self._off_val = n_gather * 4
        self._off_flags = 2 * n_gather * 4
        self._off_sent = self._off_flags + world * rows * 4
        self._off_seen = self._off_sent + rows * 4
        super().__init__(self._off_seen + rows * 4, world, rank, device)
        a = self.arena
        self.gather_idx = a[:self._off_val].view(torch.int32).view(2, rows, world, topk)
        self.gather_val = a[self._off_val:self._off_flags].view(torch.float32).view(2, rows, world, topk)
        self.flags = a[self._off_flags:self._off_sent].view(torch.int32).view(world, rows)
        self.sent = a[self._off_sent:self._off_seen].view(torch.int32)
        self.seen = a[self._off_seen:self._off_seen + rows * 4].view(torch.int32)
        self._ptr_arrays = None

    def _mapped(self) -> None:
        self._ptr_arrays = (self._peer_pointers(0), self._peer_pointers(self._off_val),
                            self._peer_pointers(self._off_flags))

    @classmethod
    def local_group(cls, rows: int, topk: int, world: int, device, wait_limit_s: float = 2.0):
        return super().local_group(rows, topk, world=world, device=device, wait_limit_s=wait_limit_s)

    # -- the two launches of a step ------------------------------------------------
    def push(self, logits: torch.Tensor, seq_lens: Optional[torch.Tensor] = None, *,
             hist: Optional[torch.Tensor] = None, index_offset: int = 0, pad_value: int = -1) -> None:
        """Local top-k of ``logits[rows, n]`` whose (position + index_offset, logit) pairs are
        stored into every rank's gather buffers, then the step is posted to every rank."""
        _need(self._ptr_arrays is not None, "call connect() (or build the ranks with local_group) first")
        _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
              "logits must be CUDA fp32 [rows, n] with dense rows")
        R, n = logits.shape
        _need(R == self.rows, f"logits has {R} rows, the exchange was built for {self.rows}")
        seq_lens = _lens(seq_lens, R)
        if hist is not None:
            _cuda_contig(hist, "hist", (torch.int32, torch.uint32))
            _need(hist.numel() == R * HIST_BINS, "hist must be [R, 4096]")
        gi, gv, fl = self._ptr_arrays
        slab_stride = logits.stride(0) if R > 1 else max(logits.stride(0), n)
        _lib.check(_lib.lib().dsa_topk_select_push(
            _ptr(logits), _ptr(seq_lens), _ptr(hist), R, n, slab_stride, self.topk, int(pad_value),
            int(index_offset), self.world, self.rank, gi, gv, fl, _ptr(self.sent), _stream()))

    def merge(self, out_idx: torch.Tensor, pad_value: int = -1) -> torch.Tensor:
        """Waits (on the device, bounded) for this step's candidates of every rank, then writes the
        exact global top-k into ``out_idx[rows, topk]``."""
        _cuda_contig(out_idx, "out_idx", (torch.int32,))
        _need(tuple(out_idx.shape) == (self.rows, self.topk), "out_idx must be [rows, topk]")
        _lib.check(_lib.lib().dsa_topk_merge_wait(
            _ptr(self.gather_idx), _ptr(self.gather_val), _ptr(self.flags), _ptr(self.seen), _ptr(out_idx),
            self.rows, self.world, self.topk, int(pad_value), self.wait_limit_ns, _stream()))
        return out_idx


class PeerAllReduce(PeerArena):
    """Sum of a small activation (up to ``max_elems`` values: the [B, hidden] output of a
    row-parallel projection at decode) over the ranks of a tensor-parallel group, as two small
    launches in stream order (``dsa_allreduce_push`` / ``dsa_allreduce_wait_sum``): capturable
    in a CUDA graph, deterministic (rank order), with a bounded wait on the device."""

    def __init__(self, max_elems: int, world: int, rank: int, device, wait_limit_s: float = 2.0) -> None:
        _need(max_elems > 0 and max_elems % 4 == 0, "max_elems must be a positive multiple of 4")
        self.max_elems = max_elems
        self.wait_limit_ns = int(wait_limit_s * 1e9)
        self._off_flags = 2 * world * max_elems * 4
        self._off_sent = self._off_flags + 64
        self._off_seen = self._off_sent + 16
        super().__init__(self._off_seen + 16, world, rank, device)
        a = self.arena
        self.flags = a[self._off_flags:self._off_flags + world * 4].view(torch.int32)
        self.sent = a[self._off_sent:self._off_sent + 4].view(torch.int32)
        self.seen = a[self._off_seen:self._off_seen + 4].view(torch.int32)
        self._ptr_arrays = None

    def _mapped(self) -> None:
        self._ptr_arrays = (self._peer_pointers(0), self._peer_pointers(self._off_flags))

    @classmethod
    def local_group(cls, max_elems: int, world: int, device, wait_limit_s: float = 2.0):
        return super().local_group(max_elems, world=world, device=device, wait_limit_s=wait_limit_s)

    def push(self, x: torch.Tensor) -> None:
        """Stores this rank's partial ``x`` (bf16 or fp32, contiguous) into every rank's slots."""
        _need(self._ptr_arrays is not None, "call connect() (or build the ranks with local_group) first")
        _cuda_contig(x, "x", (torch.bfloat16, torch.float32))
        n = x.numel()
        _need(n % 4 == 0 and n <= self.max_elems, f"x has {n} elements: a multiple of 4, at most {self.max_elems}")
        self._n = n
        slots, flags = self._ptr_arrays
        # the slot stride is the element count of THIS call: every rank passes the same shape
        _lib.check(_lib.lib().dsa_allreduce_push(_ptr(x), 1 if x.dtype == torch.bfloat16 else 0, n, self.world,
                                                 self.rank, slots, flags, _ptr(self.sent), _stream()))

    def wait_sum(self, out: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out = sum over ranks (+ residual)``, once every rank's partial of this step is there."""
        _cuda_contig(out, "out", (torch.bfloat16, torch.float32))
        n = out.numel()
        _need(n == getattr(self, "_n", n), "out must have the element count that was pushed")
        if residual is not None:
            _cuda_contig(residual, "residual", (out.dtype,))
            _need(residual.numel() == n, "residual must have out's element count")
        _lib.check(_lib.lib().dsa_allreduce_wait_sum(
            _ptr(self.arena), _ptr(self.flags), _ptr(self.seen), _ptr(residual), _ptr(out),
            1 if out.dtype == torch.bfloat16 else 0, n, self.world, self.wait_limit_ns, _stream()))
        return out

    def all_reduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.push(x)
        return self.wait_sum(torch.empty_like(x) if out is None else out, residual)
