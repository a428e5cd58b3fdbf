"""Serving-shaped entry of the hot path: one call per layer for a batch of decode
rows over the PAGED caches, graph-capturable, every buffer static-shaped.

Mirror of the reference overlay's ``_hh_fused_hide_decode_paged``
(sglang_overlay/mli-sglang-v0.5.16.patch:1282-1548): same arguments, same modes
(``"full"``, ``"attn_only"``, ``"scan_only"``), same ``select`` values and return
shapes, same conventions (outputs are VIEWS of persistent scratch keyed by the
static shape, overwritten by the next call; ``-1`` pads the selection; per-row
lengths and the page table are read on the device).

Differences a caller can observe: a bf16 ``kv_pool`` is attended in place through
the slot numbers (the reference first gathers the rows with ``index_select``);
``select="approx"`` runs the exact selection; the work is a few launches in
stream order instead of one launch with an in-kernel row barrier
(kernels/cuda_fused_sparse_splitk.py:2025-2028).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch

from . import ops

_FP8_ROW = ops.FP8_LATENT_ROW
_scratch: Dict[Tuple, torch.Tensor] = {}


def _hide_scratch(key: Tuple, make):
    """Persistent scratch keyed by static shape (patch :1274-1279): allocated on
    first use, reused by every later call and by graph replays."""
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = make()
    return buf


def clear_scratch() -> None:
    _scratch.clear()


def fused_hide_decode_paged(
    q_all: torch.Tensor,
    kv_pool: torch.Tensor,
    incumbent_slots: torch.Tensor,
    index_q_fp8: torch.Tensor,
    index_weights: torch.Tensor,
    index_k_paged: torch.Tensor,
    page_table: torch.Tensor,
    seq_lens: torch.Tensor,
    skv_cap: int,
    sm_scale: float,
    out_index_pool: Optional[torch.Tensor],
    nsplit: Optional[int] = None,
    index_topk: Optional[int] = None,
    nsplit_attn: Optional[int] = None,
    return_logits: bool = False,
    select: Union[bool, str] = True,
    mode: str = "full",
):
    """Attention over each row's incumbent KV slots + this layer's FP8 indexer over
    the row's full paged prefix -> next index set (patch :1352-1366 for the
    arguments). Returns, as the reference does (:1518-1548): ``attn_out
    [1,B,H,512]`` for ``mode="attn_only"``; the ``[B, skv_cap]`` logit slab for
    ``"scan_only"``; for ``"full"``: ``(attn_out, logits)`` under
    ``select=False/"prod"``, ``(attn_out, next_idx int32 [B, topk])`` under
    ``select=True/"kernel"/"exact"/"approx"`` (KV-slot space, ``-1`` padded;
    plus ``logits`` with ``return_logits``), ``(attn_out, next_idx int64)`` under
    ``select="torch"`` (torch.topk gate)."""
    if mode not in ("full", "attn_only", "scan_only"):
        raise ValueError(f"unknown mode={mode!r}")
    if select is True:
        sel_mode = "exact"
    elif select is False:
        sel_mode = "prod"
    else:
        sel_mode = "exact" if select in ("kernel", "approx") else str(select)
    if sel_mode == "prod_side":
        sel_mode = "prod"  # the side-stream placement is the caller's business
    if sel_mode not in ("exact", "prod", "torch"):
        raise ValueError(f"unknown select={select!r}")
    if q_all.dim() != 4 or q_all.shape[0] != 1:
        raise ValueError(f"q_all must be [1,B,H,dqk], got {tuple(q_all.shape)}")
    _, B, H_real, dqk = q_all.shape
    device = q_all.device
    if dqk != ops.LATENT_DIM:
        raise ValueError(f"dqk must be {ops.LATENT_DIM}, got {dqk}")
    if index_q_fp8.dim() != 3 or index_q_fp8.shape[0] != B:
        raise ValueError(f"index_q_fp8 must be [B={B},Hidx,didx], got {tuple(index_q_fp8.shape)}")
    Hidx, didx = int(index_q_fp8.shape[1]), int(index_q_fp8.shape[2])
    if didx != ops.INDEX_DIM or Hidx % 16:
        raise ValueError(f"unsupported indexer geometry Hidx={Hidx} didx={didx}")
    if index_q_fp8.dtype not in (torch.float8_e4m3fn, torch.uint8):
        raise ValueError(f"index_q_fp8 dtype {index_q_fp8.dtype}")
    if tuple(index_weights.shape) != (B, Hidx):
        raise ValueError(f"index_weights must be [B,Hidx]=({B},{Hidx}), got {tuple(index_weights.shape)}")
    if tuple(seq_lens.shape) != (B,) or seq_lens.dtype != torch.int32:
        raise ValueError(f"seq_lens must be int32 [B={B}], got {tuple(seq_lens.shape)} {seq_lens.dtype}")
    if page_table.dim() != 2 or page_table.shape[0] != B or page_table.dtype != torch.int32:
        raise ValueError(f"page_table must be int32 [B={B}, pt_stride], got {tuple(page_table.shape)} {page_table.dtype}")
    pt_stride = int(page_table.shape[1])
    skv_cap = int(skv_cap)
    if pt_stride * ops.PAGE_TOKENS < skv_cap:
        raise ValueError(f"page table ({pt_stride} pages) does not cover skv_cap={skv_cap}")
    if index_k_paged.dtype != torch.uint8 or index_k_paged.dim() != 2 or index_k_paged.shape[1] != ops.INDEX_PAGE_BYTES:
        raise ValueError(f"index_k_paged must be uint8 [num_pages, {ops.INDEX_PAGE_BYTES}]")
    if out_index_pool is not None and (out_index_pool.shape[0] != B or out_index_pool.shape[1] < skv_cap):
        raise ValueError(f"out_index_pool must be [B={B}, >= {skv_cap}], got {tuple(out_index_pool.shape)}")
    if incumbent_slots.shape[0] != B:
        raise ValueError(f"incumbent batch {incumbent_slots.shape[0]} != {B}")
    topk = int(incumbent_slots.shape[1])
    index_topk = topk if index_topk is None else int(index_topk)
    S_pool, row_w = kv_pool.shape
    kv_fp8 = row_w == _FP8_ROW and kv_pool.dtype in (torch.uint8, torch.float8_e4m3fn)
    if not kv_fp8 and not (row_w == dqk and kv_pool.dtype == torch.bfloat16):
        raise ValueError(f"kv_pool must be bf16 [S,{dqk}] or fp8-packed uint8 [S,{_FP8_ROW}], got "
                         f"{kv_pool.dtype} {tuple(kv_pool.shape)}")

    # Head-geometry convention of the reference (:1443-1452): pad the heads to a multiple
    # of 16 with zero queries (a persistent buffer) and slice them off on return.
    H = (H_real + 15) // 16 * 16
    if H != H_real:
        qpad = _hide_scratch((str(device), B, H, "qpad"),
                             lambda: torch.zeros(1, B, H, dqk, dtype=torch.bfloat16, device=device))
        qpad[:, :, :H_real].copy_(q_all)
        q_all = qpad
    q = q_all.contiguous().view(B, H, dqk)
    if nsplit_attn is None:
        nsplit_attn = nsplit if nsplit is not None else ops.default_nsplit(B, H, topk)
    nsplit_attn = int(nsplit_attn)
    key = (str(device), B, H, skv_cap, nsplit_attn, topk)

    attn_out = logits = None
    if mode != "scan_only":
        # one shared pool of S_pool slots: every row is a query row of the same "sequence",
        # entries < 0 or >= S_pool are skipped in the kernel
        slots = incumbent_slots if incumbent_slots.dtype == torch.int32 else incumbent_slots.to(torch.int32)
        kv = (kv_pool if kv_pool.dtype != torch.float8_e4m3fn else kv_pool.view(torch.uint8)).unsqueeze(0)
        scratch = _hide_scratch(key + ("part",), lambda: ops.MlaScratch(B, H, nsplit_attn, device))
        out = _hide_scratch(key + ("out",), lambda: torch.zeros(1, B, H, ops.VALUE_DIM, dtype=torch.bfloat16,
                                                                 device=device))
        ops.sparse_mla_decode(q, kv, slots.contiguous(), float(sm_scale), None, rows_per_seq=B, nsplit=nsplit_attn,
                              scratch=scratch, out=out.view(B, H, ops.VALUE_DIM))
        attn_out = out[:, :, :H_real] if H != H_real else out
        if mode == "attn_only":
            return attn_out

    slab = _hide_scratch(key + ("slab",), lambda: torch.empty(B, (skv_cap + 3) // 4 * 4, dtype=torch.float32,
                                                              device=device))
    use_hist = mode == "full" and sel_mode == "exact"
    hist = _hide_scratch(key + ("hist",), lambda: torch.zeros(B, ops.HIST_BINS, dtype=torch.int32, device=device))
    iq = index_q_fp8 if index_q_fp8.dtype == torch.uint8 else index_q_fp8.view(torch.uint8)
    ops.indexer_scan_fp8_paged(iq.contiguous(), index_weights.to(torch.float32).contiguous(), index_k_paged,
                               page_table.contiguous(), seq_lens.contiguous(), skv_cap, out=slab,
                               hist=hist if use_hist else None)
    logits = slab[:, :skv_cap]
    if mode == "scan_only":
        return logits
    if sel_mode == "prod":
        return attn_out, logits

    if sel_mode == "exact":
        if index_topk != topk:
            raise ValueError("the in-launch select emits exactly topk indices")
        ws = _hide_scratch(key + ("topk_ws",), lambda: ops.topk_workspace(B, skv_cap, device))
        pos = _hide_scratch(key + ("pos",), lambda: torch.full((B, topk), -1, dtype=torch.int32, device=device))
        next_idx = _hide_scratch(key + ("nextidx",), lambda: torch.full((B, topk), -1, dtype=torch.int32,
                                                                        device=device))
        ops.topk_select(logits, topk, seq_lens, hist=hist, out_idx=pos, workspace=ws)
        # positions -> KV slots: through out_index_pool, or page * 64 + offset from the page-64
        # table (kernels/cuda_fused_sparse_splitk.py:1142-1144); padding stays -1
        safe = pos.clamp(min=0).long()
        if out_index_pool is not None:
            mapped = torch.gather(out_index_pool[:, :skv_cap], 1, safe).to(torch.int32)
        else:
            mapped = torch.gather(page_table, 1, safe >> 6) * ops.PAGE_TOKENS + (pos & (ops.PAGE_TOKENS - 1))
        torch.where(pos >= 0, mapped, pos, out=next_idx)
        if return_logits:
            return attn_out, next_idx, logits
        return attn_out, next_idx

    # torch top-k over the full-prefix logits (gate only, :1531-1548)
    if out_index_pool is None:
        raise ValueError("select='torch' needs out_index_pool")
    k = min(index_topk, skv_cap)
    top_v, top_pos = torch.topk(logits, k, dim=-1)
    next_idx = torch.gather(out_index_pool.long()[:, :skv_cap], 1, top_pos)
    next_idx = torch.where(torch.isfinite(top_v), next_idx, torch.full_like(next_idx, -1))
    if k < index_topk:
        next_idx = torch.cat([next_idx, torch.full((B, index_topk - k), -1, dtype=next_idx.dtype, device=device)], 1)
    if return_logits:
        return attn_out, next_idx, logits.clone()
    return attn_out, next_idx


def forward_hide_operands(
    q_proj: torch.Tensor,
    k_proj: torch.Tensor,
    head_gates: torch.Tensor,
    k_norm_weight: torch.Tensor,
    k_norm_bias: torch.Tensor,
    k_norm_eps: float,
    rope_cos: torch.Tensor,
    rope_sin: torch.Tensor,
    positions: torch.Tensor,
    index_k_paged: torch.Tensor,
    page_table_64: torch.Tensor,
    seq_lens: torch.Tensor,
    rope_interleave: bool = False,
    scale_fmt: Optional[str] = None,
    softmax_scale: Optional[float] = None,
):
    """This layer's indexer PREPARE + STORE without a top-k, for a batch of decode
    rows: the operands ``fused_hide_decode_paged`` scans with. Counterpart of the
    overlay's ``Indexer.forward_hide_operands`` after its projections
    (sglang_overlay/mli-sglang-v0.5.16.patch:252-363, non-fusion branch :322-342):
    ``q_proj`` = wq_b(q_lora) ``[B, Hidx, 128]`` bf16, ``k_proj`` = wk(x) ``[B, 128]``
    bf16, ``head_gates`` = weights_proj(x) ``[B, Hidx]`` fp32 (not yet scaled). One
    launch rotates, quantises, folds ``n_heads^-0.5 * q_scale * softmax_scale`` into
    the gates and stores each row's key at ``positions[b]`` in its page.

    Returns the reference's tuple ``(q_fp8 [B,Hidx,128] uint8 bytes, weights [B,Hidx]
    fp32, index_k_paged, page_table_64 int32, seq_lens int32, skv_cap)``; the first
    two are views of persistent scratch keyed by the static shape (graph-capturable:
    no host integer is read from the device). Raises where the reference refuses to
    engage (:279-312): page size other than 64, missing table or lengths."""
    if page_table_64 is None or seq_lens is None:
        raise RuntimeError("[HIDE VOID] page-64 table / int32 seqlens unavailable")
    if index_k_paged.dim() != 2 or index_k_paged.shape[1] != ops.INDEX_PAGE_BYTES:
        raise RuntimeError(f"[HIDE VOID] index-K pages must be [num_pages, {ops.INDEX_PAGE_BYTES}] "
                           "(64-token pages)")
    if page_table_64.dtype != torch.int32:
        page_table_64 = page_table_64.to(torch.int32)
    if seq_lens.dtype != torch.int32:
        seq_lens = seq_lens.to(torch.int32)
    B, n_heads = q_proj.shape[0], q_proj.shape[1]
    device = q_proj.device
    q_fp8 = _hide_scratch(("hide_q", B, n_heads, device),
                          lambda: torch.empty(B, n_heads, ops.INDEX_DIM, dtype=torch.uint8, device=device))
    weights = _hide_scratch(("hide_w", B, n_heads, device),
                            lambda: torch.empty(B, n_heads, dtype=torch.float32, device=device))
    ops.indexer_stage_fp8(q_proj, k_proj, head_gates, k_norm_weight, k_norm_bias, k_norm_eps, rope_cos, rope_sin,
                          positions, q_fp8, weights, pages=index_k_paged.view(-1), page_table=page_table_64,
                          rope_interleave=rope_interleave, scale_fmt=scale_fmt, softmax_scale=softmax_scale)
    skv_cap = int(page_table_64.shape[1]) * ops.PAGE_TOKENS
    return q_fp8, weights, index_k_paged, page_table_64, seq_lens, skv_cap


_hh_fused_hide_decode_paged = fused_hide_decode_paged  # the reference's name for it
