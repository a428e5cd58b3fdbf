"""The reference kernel extension's launch functions, same names and argument
lists, on top of libdsa_b200.so.

The reference builds a torch extension and calls
``ext.launch_fused_sparse_splitk(...)``, ``..._batch_idx(...)`` and
``..._paged(...)`` (kernels/cuda_fused_sparse_splitk.py:2634-2655, :2744-2760,
:2770-2808). ``build()`` here returns an object with those three entry points
so the reference's callers (inference/modeling/transformer.py:3071-3234, the
SGLang overlay's hh_fused_decode.py) can bind to it unchanged. What one launch
does there is a pair of launches here: the attention half
(``attn_on``) and the indexer half (``with_select`` 1 or 2).

Differences a caller can observe: PartAcc/PartM/PartL are used as
``[S, nsplit, H, 512]`` / ``[S, nsplit, H]`` scratch (same element count, other
order); ``SelHist`` (``with_select == 2``) must be ``[S, 4096]`` int32, the
12-bit histogram ``dsa_topk_select`` consumes, instead of the reference's 256
bins; the tap/cascade modes (``with_select >= 3``, ``win``) are not provided.
"""

from __future__ import annotations

import torch

from . import _lib, ops

_DQK, _DV, _DIDX = 576, 512, 128


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


_LENS = {}


def _causal_lens(S: int, Skv: int, device) -> torch.Tensor:
    """Visible keys of each of the S query rows of one sequence (row s sees Skv - S + s + 1),
    built once per (S, Skv, device): a launch then allocates nothing and stays capturable."""
    key = (S, Skv, str(device))
    lens = _LENS.get(key)
    if lens is None:
        lens = _LENS[key] = torch.arange(Skv - S + 1, Skv + 1, dtype=torch.int32, device=device)
    return lens


def _check_modes(with_select: int, win: int) -> None:
    if with_select not in (0, 1, 2):
        raise RuntimeError("with_select >= 3 (tap cascade) is not provided by this build")
    if win not in (0, None):
        raise RuntimeError("the admission window (win) belongs to the tap cascade and is not provided")


class FusedSparseSplitK:
    """Object returned by :func:`build`; its methods mirror the extension's functions."""

    def launch_fused_sparse_splitk(self, Q, KV, Indices, IndexQ, IndexK, IndexW, IndexKScale, PartAcc, PartM,
                                   PartL, SelSlab, SelHist, Out, S, Skv, H, Hidx, topk, nsplit, sm_scale,
                                   with_select, attn_on, win):
        """One sequence, S query rows; row s sees keys [0, Skv - S + s]."""
        _check_modes(with_select, win)
        lib = _lib.lib()
        lens = _causal_lens(S, Skv, Q.device)
        if attn_on:
            _lib.check(lib.dsa_sparse_mla_decode(_p(Q), _p(KV), _p(Indices), _p(lens), _p(PartAcc), _p(PartM),
                                                 _p(PartL), _p(Out), S, S, H, topk, nsplit, float(sm_scale), Skv, 0,
                                                 _st()))
        if with_select:
            hist = SelHist if with_select == 2 else None
            _lib.check(lib.dsa_indexer_scan_fp8(_p(IndexQ), _p(IndexW), _p(IndexK), _p(IndexKScale), _p(lens),
                                                _p(SelSlab), _p(hist), S, S, Hidx, Skv, 1, Skv, Skv, Skv, 0, _st()))

    def launch_fused_sparse_splitk_batch_idx(self, Q, KV, Indices, IndexQ, IndexK, IndexW, IndexKScale, PartAcc,
                                             PartM, PartL, SelSlab, SelHist, Out, S, Skv, H, Hidx, topk, nsplit,
                                             sm_scale, with_select, attn_on, win, kv_stride, idx_k_stride,
                                             idx_scale_stride):
        """S independent sequences, one query row each; strides are in elements
        (reference :533-535); every row sees its whole prefix of Skv keys."""
        _check_modes(with_select, win)
        if kv_stride % _DQK or idx_k_stride % _DIDX:
            raise RuntimeError("kv_stride / idx_k_stride must be whole rows")
        lib = _lib.lib()
        if attn_on:
            _lib.check(lib.dsa_sparse_mla_decode(_p(Q), _p(KV), _p(Indices), None, _p(PartAcc), _p(PartM), _p(PartL),
                                                 _p(Out), S, 1, H, topk, nsplit, float(sm_scale), kv_stride // _DQK,
                                                 0, _st()))
        if with_select:
            hist = SelHist if with_select == 2 else None
            _lib.check(lib.dsa_indexer_scan_fp8(_p(IndexQ), _p(IndexW), _p(IndexK), _p(IndexKScale), None,
                                                _p(SelSlab), _p(hist), S, 1, Hidx, Skv, S, idx_k_stride // _DIDX,
                                                idx_scale_stride, Skv, 0, _st()))

    def launch_fused_sparse_splitk_paged(self, Q, KV, Indices, IndexQ, IndexKPaged, IndexW, SeqLens, PageTable,
                                         PartAcc, PartM, PartL, SelSlab, SelHist, Out, S, Skv, H, Hidx, topk, nsplit,
                                         sm_scale, with_select, attn_on, kv_stride, pt_stride, page_bytes,
                                         slab_stride, nsplit_attn, kv_fp8, kv_rows, sel_on, SelScratch, NextIdx,
                                         sel_m):
        """Serving form: page-64 index keys, device-side lengths, optional fp8
        latent pool addressed by KV-slot indices (entries < 0 are skipped)."""
        _check_modes(with_select, 0)
        if page_bytes != ops.INDEX_PAGE_BYTES:
            raise RuntimeError(f"page_bytes must be {ops.INDEX_PAGE_BYTES}")
        lib = _lib.lib()
        n_att = nsplit_attn if nsplit_attn and nsplit_attn > 0 else nsplit
        if attn_on:
            if kv_fp8:  # one shared pool of kv_rows slots; Indices are slot numbers
                _lib.check(lib.dsa_sparse_mla_decode(_p(Q), _p(KV), _p(Indices), None, _p(PartAcc), _p(PartM),
                                                     _p(PartL), _p(Out), S, S, H, topk, n_att, float(sm_scale),
                                                     kv_rows, 1, _st()))
            else:
                _lib.check(lib.dsa_sparse_mla_decode(_p(Q), _p(KV), _p(Indices), _p(SeqLens), _p(PartAcc), _p(PartM),
                                                     _p(PartL), _p(Out), S, 1, H, topk, n_att, float(sm_scale),
                                                     kv_stride // _DQK, 0, _st()))
        if with_select:
            hist = SelHist if (with_select == 2 or sel_on) else None
            slab = slab_stride if slab_stride and slab_stride > 0 else Skv
            _lib.check(lib.dsa_indexer_scan_fp8_paged(_p(IndexQ), _p(IndexW), _p(IndexKPaged), IndexKPaged.shape[0],
                                                      _p(PageTable), pt_stride, _p(SeqLens), _p(SelSlab), _p(hist),
                                                      S, Hidx, Skv, slab, _st()))
            if sel_on:  # in-launch selection: SelScratch is the top-k workspace, NextIdx the result
                _lib.check(lib.dsa_topk_select(_p(SelSlab), _p(SeqLens), _p(hist), None, _p(NextIdx), None,
                                               _p(SelScratch), SelScratch.numel() * SelScratch.element_size(), S, Skv,
                                               slab, topk, -1, 0, _st()))


def build() -> FusedSparseSplitK:
    """Counterpart of the reference's ``build()`` (kernels/cuda_fused_sparse_splitk.py:2922-2941):
    loads the prebuilt sm_100a library instead of JIT-compiling."""
    _lib.lib()
    return FusedSparseSplitK()


def alloc_part(S: int, H: int, nsplit: int, dev):
    """Split-K scratch with the reference's element counts (:3005-3009)."""
    nb = S * (H // 16) * nsplit
    return (torch.zeros(nb, 16, _DV, dtype=torch.float32, device=dev),
            torch.zeros(nb, 16, dtype=torch.float32, device=dev),
            torch.zeros(nb, 16, dtype=torch.float32, device=dev))
