"""One DSA transformer block on the GPU, with the reference's layer API.

Same module tree, parameter names and construction order as the reference's
``DSALayer`` (src/lagged_indexer_dsa/dsa_layer.py:55-196), so a ``state_dict``
(or a seed) gives identical weights in both. The projections, norms, RoPE and
the SwiGLU MLP are torch ops (cuBLAS GEMV/GEMM); the three hot operations --
indexer logits, top-k selection, sparse MLA -- go to the CUDA library:

* production geometry (576-wide latent, 128-wide index keys) in bf16: FP8
  tcgen05 scan, exact top-k, split-K bf16 attention;
* any other geometry or fp32 weights: the library's fp32 kernels, which follow
  the reference arithmetic (attention_core.py:27-160) to ~1e-5.

Beside the reference's full-sequence methods there is a decode form
(``decode_project`` / ``decode_indexer`` / ``decode_attention``) over per-layer
caches, which the reference layer lacks.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple


import torch
from torch import nn

from . import ops
from .config import DSAConfig
from .rope import apply_rotary, apply_rotary_at


@dataclasses.dataclass
class RopeCaches:
    """Rotary tables shared by all layers (reference dsa_layer.py:32-39)."""

    mla_cos: torch.Tensor
    mla_sin: torch.Tensor
    idx_cos: torch.Tensor
    idx_sin: torch.Tensor


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor):
        """``(x + delta, self(x + delta))``: the residual addition and this norm, one
        launch for bf16 rows on a CUDA device, two separate steps otherwise."""
        if (x.is_cuda and x.dtype == torch.bfloat16 and delta.dtype == torch.bfloat16 and x.shape == delta.shape
                and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192 and not torch.is_grad_enabled()):
            return ops.add_rmsnorm(x, delta, self.weight, self.eps)
        s = x + delta
        return s, self(s)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16):
            return ops.rmsnorm(x, self.weight, self.eps)  # one launch
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * inv * self.weight.float()).to(x.dtype)


@dataclasses.dataclass
class LayerDecodeCache:
    """Decode caches of one layer for ``n_seq`` sequences of capacity ``cap``.

    fp8 mode: index_k e4m3 ``[n_seq, cap, 128]`` + k_scale fp32, kv bf16
    ``[n_seq, cap, 576]``. fp32 mode: index_k and kv are fp32 of any width."""

    index_k: torch.Tensor
    k_scale: Optional[torch.Tensor]
    kv: torch.Tensor

    @property
    def capacity(self) -> int:
        return self.kv.shape[1]


@dataclasses.dataclass
class IndexerWorkspace:
    """Persistent buffers of one layer's decode indexer: logits slab, the scan's
    histogram (zero once, re-armed by the select), top-k scratch and result."""

    logits: torch.Tensor
    hist: Optional[torch.Tensor]
    topk_ws: torch.Tensor
    indices: torch.Tensor

    @staticmethod
    def create(n_seq: int, capacity: int, topk: int, device, fp8: bool) -> "IndexerWorkspace":
        slab = (capacity + 3) // 4 * 4
        return IndexerWorkspace(
            torch.empty(n_seq, slab, dtype=torch.float32, device=device),
            torch.zeros(n_seq, ops.HIST_BINS, dtype=torch.int32, device=device) if fp8 else None,
            ops.topk_workspace(n_seq, capacity, device),
            torch.full((n_seq, topk), -1, dtype=torch.int32, device=device))


def _pad_heads(t: torch.Tensor, multiple: int) -> torch.Tensor:
    """Zero-pads dim 1 (heads) to a multiple; zero queries attend uniformly and
    are dropped by the caller (reference fused_decode.py:38-43)."""
    h = t.shape[1]
    extra = (-h) % multiple
    if extra == 0:
        return t
    pad = torch.zeros(t.shape[0], extra, *t.shape[2:], dtype=t.dtype, device=t.device)
    return torch.cat([t, pad], dim=1)


class DSALayer(nn.Module):
    def __init__(self, config: DSAConfig) -> None:
        super().__init__()
        self.config = config
        c = config
        h = c.num_attention_heads
        self.attn_norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.ffn_norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        # MLA query path
        self.q_a_proj = nn.Linear(c.hidden_size, c.q_lora_rank, bias=False)
        self.q_a_layernorm = RMSNorm(c.q_lora_rank, c.rms_norm_eps)
        self.q_b_proj = nn.Linear(c.q_lora_rank, h * (c.qk_nope_head_dim + c.qk_rope_head_dim), bias=False)
        # MLA key/value path
        self.kv_a_proj = nn.Linear(c.hidden_size, c.kv_lora_rank + c.qk_rope_head_dim, bias=False)
        self.kv_a_layernorm = RMSNorm(c.kv_lora_rank, c.rms_norm_eps)
        self.kv_b_proj = nn.Linear(c.kv_lora_rank, h * (c.qk_nope_head_dim + c.v_head_dim), bias=False)
        self.o_proj = nn.Linear(h * c.v_head_dim, c.hidden_size, bias=False)
        # lightning indexer
        self.index_q_proj = nn.Linear(c.q_lora_rank, c.index_n_heads * c.index_head_dim, bias=False)
        self.index_k_proj = nn.Linear(c.hidden_size, c.index_head_dim, bias=False)
        self.index_weights_proj = nn.Linear(c.q_lora_rank, c.index_n_heads, bias=False)
        # SwiGLU MLP
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)
        # Set by DSAModel.tensor_parallel: this module then holds one rank's heads and MLP columns,
        # and the outputs of o_proj / down_proj are partial sums that `tp.reduce` completes.
        self.tp = None

    def _reduced(self, partial: torch.Tensor) -> torch.Tensor:
        return partial if self.tp is None else self.tp.reduce(partial)

    # ------------------------------------------------------------------ helpers
    def _fast_path(self, t: torch.Tensor) -> bool:
        """True when the FP8/bf16 tensor-core kernels apply to tensors like ``t``."""
        return self.config.is_production_geometry and t.dtype == torch.bfloat16

    @property
    def sm_scale(self) -> float:
        # the reference layer uses sparse_mla_core's default D_qk ** -0.5 (attention_core.py:141-142)
        return self.config.qk_head_dim ** -0.5

    def _w_uk_uv(self) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self.config
        w = self.kv_b_proj.weight.view(c.num_attention_heads, c.qk_nope_head_dim + c.v_head_dim, c.kv_lora_rank)
        return w[:, : c.qk_nope_head_dim, :], w[:, c.qk_nope_head_dim:, :]

    # ------------------------------------------------------------------ stacked decode projections
    def fuse_decode_weights(self) -> None:
        """Stacks the weights of the three projections that read x_norm (q_a, kv_a,
        index_k) and of the three that read c_q (q_b, index_q, index_weights), so a
        decode step needs two GEMVs instead of six small launches. The parameters
        become views of the stacked tensors: no extra memory, ``state_dict`` and
        ``load_state_dict`` keep working, and moving or casting the module afterwards
        simply drops the stacking (``decode_project`` notices and uses the six)."""
        with torch.no_grad():
            for name, mods in (("_wx", (self.q_a_proj, self.kv_a_proj, self.index_k_proj)),
                               ("_wc", (self.q_b_proj, self.index_q_proj, self.index_weights_proj))):
                stacked = torch.cat([m.weight for m in mods], dim=0)
                row = 0
                for m in mods:
                    n = m.weight.shape[0]
                    m.weight.data = stacked[row:row + n]
                    row += n
                setattr(self, name, stacked)

    def _stacked(self) -> bool:
        wx, wc = getattr(self, "_wx", None), getattr(self, "_wc", None)
        return (wx is not None and wc is not None and self.q_a_proj.weight.data_ptr() == wx.data_ptr()
                and self.q_b_proj.weight.data_ptr() == wc.data_ptr()
                and self.index_k_proj.weight.data_ptr() == wx[wx.shape[0] - self.index_k_proj.weight.shape[0]:].data_ptr()
                and self.index_weights_proj.weight.data_ptr()
                == wc[wc.shape[0] - self.index_weights_proj.weight.shape[0]:].data_ptr())

    # ------------------------------------------------------------------ projections (torch)
    def q_latent(self, x_norm: torch.Tensor) -> torch.Tensor:
        """c_q = q_a_layernorm(q_a_proj(x_norm)), shared by attention and indexer."""
        return self.q_a_layernorm(self.q_a_proj(x_norm))

    def _mla_qkv(self, x_norm, c_q, rope: RopeCaches):
        c = self.config
        b, s, _ = x_norm.shape
        h = c.num_attention_heads
        q = self.q_b_proj(c_q).view(b, s, h, c.qk_nope_head_dim + c.qk_rope_head_dim)
        q_nope, q_rope = q.split([c.qk_nope_head_dim, c.qk_rope_head_dim], dim=-1)
        q_rope = apply_rotary(q_rope.transpose(1, 2), rope.mla_cos, rope.mla_sin).transpose(1, 2)
        kv_a = self.kv_a_proj(x_norm)
        c_kv, k_rope = kv_a.split([c.kv_lora_rank, c.qk_rope_head_dim], dim=-1)
        c_kv = self.kv_a_layernorm(c_kv)
        k_rope = apply_rotary(k_rope.unsqueeze(1), rope.mla_cos, rope.mla_sin).squeeze(1)
        w_uk, _ = self._w_uk_uv()
        q_abs = torch.einsum("bshd,hdl->bshl", q_nope, w_uk)  # absorb W_UK into the query
        return torch.cat([q_abs, q_rope], dim=-1), torch.cat([c_kv, k_rope], dim=-1)

    def _project_output(self, o_latent: torch.Tensor) -> torch.Tensor:
        c = self.config
        _, w_uv = self._w_uk_uv()
        o = torch.einsum("bshl,hdl->bshd", o_latent, w_uv)
        return self._reduced(self.o_proj(o.reshape(o.shape[0], o.shape[1], c.num_attention_heads * c.v_head_dim)))

    def _indexer_qkw(self, x_norm, c_q, rope: RopeCaches):
        c = self.config
        b, s, _ = x_norm.shape
        il = c.indexer_rope_interleave
        iq = self.index_q_proj(c_q).view(b, s, c.index_n_heads, c.index_head_dim)
        iq = apply_rotary(iq.transpose(1, 2), rope.idx_cos, rope.idx_sin, interleave=il).transpose(1, 2)
        ik = apply_rotary(self.index_k_proj(x_norm).unsqueeze(1), rope.idx_cos, rope.idx_sin, interleave=il).squeeze(1)
        return iq, ik, self.index_weights_proj(c_q)

    # ------------------------------------------------------------------ hot ops (CUDA library)
    @staticmethod
    def _causal_lens(b: int, s: int, device) -> torch.Tensor:
        return torch.arange(1, s + 1, dtype=torch.int32, device=device).repeat(b)

    def _select(self, iq, ik, w, seq_lens, rows_per_seq: int, pad_value: int) -> torch.Tensor:
        """Top-k key positions per query row. iq [R,H,D], ik [n_seq,N,D], w [R,H]."""
        topk = self.config.index_topk
        if self._fast_path(iq):
            iq8, sq = ops.quantize_e4m3_rowwise(iq.float().contiguous())
            ik8, sk = ops.quantize_e4m3_rowwise(ik.float().contiguous())
            logits = ops.indexer_scan_fp8(iq8, (sq * w.float()).contiguous(), ik8, sk, seq_lens,
                                          rows_per_seq=rows_per_seq)
        else:
            logits = ops.indexer_scan_f32(iq.float().contiguous(), w.float().contiguous(), ik.float().contiguous(),
                                          seq_lens, rows_per_seq=rows_per_seq)
        return ops.topk_select(logits, topk, seq_lens, pad_value=pad_value)

    def _attend(self, q, kv, indices, seq_lens, rows_per_seq: int) -> torch.Tensor:
        """Latent attention output [R,H,Dv]. q [R,H,Dqk], kv [n_seq,N,Dqk]; indices int32 or None (dense)."""
        c = self.config
        if self._fast_path(q):
            h = q.shape[1]
            out = ops.sparse_mla_decode(_pad_heads(q, ops.HEAD_BLOCK).contiguous(), kv.contiguous(), indices,
                                        self.sm_scale, seq_lens, rows_per_seq=rows_per_seq)
            return out[:, :h]
        out = ops.sparse_mla_f32(q.float().contiguous(), kv.float().contiguous(), indices, c.kv_lora_rank,
                                 self.sm_scale, seq_lens, rows_per_seq=rows_per_seq)
        return out.to(q.dtype)

    # ------------------------------------------------------------------ reference API (full sequence)
    def indexer_indices(self, x_norm, rope: RopeCaches, c_q=None) -> torch.Tensor:
        """int64 [B,S,topk] selected key positions, padded with S (reference :145-153)."""
        if c_q is None:
            c_q = self.q_latent(x_norm)
        iq, ik, w = self._indexer_qkw(x_norm, c_q, rope)
        b, s = x_norm.shape[0], x_norm.shape[1]
        lens = self._causal_lens(b, s, x_norm.device)
        idx = self._select(iq.reshape(b * s, *iq.shape[2:]), ik, w.reshape(b * s, -1), lens, s, pad_value=s)
        return idx.view(b, s, -1).long()

    def attention_output(self, x_norm, rope: RopeCaches, indices, c_q=None) -> torch.Tensor:
        """Attention hidden output; ``indices=None`` is dense causal (reference :156-171)."""
        if c_q is None:
            c_q = self.q_latent(x_norm)
        q, kv = self._mla_qkv(x_norm, c_q, rope)
        b, s, h = q.shape[0], q.shape[1], q.shape[2]
        lens = self._causal_lens(b, s, x_norm.device)
        idx32 = None if indices is None else indices.reshape(b * s, -1).to(torch.int32).contiguous()
        o = self._attend(q.reshape(b * s, h, -1), kv, idx32, lens, s)
        return self._project_output(o.view(b, s, h, -1))

    def fused_attention_and_indices(self, x_norm, rope: RopeCaches, attn_indices, produce_indexer: bool = True):
        """One shared query latent for both consumers (reference :173-192)."""
        c_q = self.q_latent(x_norm)
        attn_hidden = self.attention_output(x_norm, rope, attn_indices, c_q=c_q)
        nxt = self.indexer_indices(x_norm, rope, c_q=c_q) if produce_indexer else None
        return attn_hidden, nxt

    def mlp(self, h_norm: torch.Tensor) -> torch.Tensor:
        if (h_norm.is_cuda and h_norm.dtype == torch.bfloat16 and h_norm.dim() == 2 and h_norm.shape[0] <= 2
                and not torch.is_grad_enabled()):
            gate, up = ops.gemv(h_norm, self.gate_proj.weight), ops.gemv(h_norm, self.up_proj.weight)
            return self._reduced(self.down_proj(ops.silu_mul(gate, up)))
        gate, up = self.gate_proj(h_norm), self.up_proj(h_norm)
        if gate.is_cuda and gate.dtype == torch.bfloat16 and not torch.is_grad_enabled():
            return self._reduced(self.down_proj(ops.silu_mul(gate, up)))  # one launch instead of two
        return self._reduced(self.down_proj(torch.nn.functional.silu(gate) * up))

    # ------------------------------------------------------------------ decode form
    def new_cache(self, n_seq: int, capacity: int, device, fp8: bool) -> LayerDecodeCache:
        c = self.config
        if fp8:
            return LayerDecodeCache(
                torch.zeros(n_seq, capacity, c.index_head_dim, dtype=torch.uint8, device=device),
                torch.zeros(n_seq, capacity, dtype=torch.float32, device=device),
                torch.zeros(n_seq, capacity, c.qk_head_dim, dtype=torch.bfloat16, device=device))
        return LayerDecodeCache(
            torch.zeros(n_seq, capacity, c.index_head_dim, dtype=torch.float32, device=device), None,
            torch.zeros(n_seq, capacity, c.qk_head_dim, dtype=torch.float32, device=device))

    def fill_cache(self, cache: LayerDecodeCache, x_norm: torch.Tensor, rope: RopeCaches) -> None:
        """Writes the keys of a whole prefix x_norm [B,S,hidden] (prefill)."""
        c_q = self.q_latent(x_norm)
        _, kv = self._mla_qkv(x_norm, c_q, rope)
        _, ik, _ = self._indexer_qkw(x_norm, c_q, rope)
        s = x_norm.shape[1]
        cache.kv[:, :s] = kv.to(cache.kv.dtype)
        if cache.k_scale is not None:
            ik8, sk = ops.quantize_e4m3_rowwise(ik.float().contiguous())
            cache.index_k[:, :s] = ik8.view(torch.uint8)
            cache.k_scale[:, :s] = sk
        else:
            cache.index_k[:, :s] = ik.float()

    def decode_project(self, x_norm, rope: RopeCaches, positions, cache: LayerDecodeCache, batch_index):
        """Projections of one new token per sequence, and its keys appended to
        the caches at ``positions`` [B]. Returns (q [B,H,Dqk], index_q, index_w).

        With FP8 caches and bf16 weights everything after the GEMVs (RoPE, e4m3
        quantisation with the scale folded into the head weights, both cache
        appends, assembly of the absorbed query) is ONE launch; index_q then
        comes back already quantised (uint8) with index_w fp32."""
        c = self.config
        b = x_norm.shape[0]
        h = c.num_attention_heads
        il = c.indexer_rope_interleave
        if self._stacked():  # two GEMVs: everything that reads x_norm, then everything that reads c_q
            # few output rows, long rows: the library GEMV is latency-bound there (measured 19-32 us
            # against 13 us for the skinny kernel at one token); the other shapes stay with the library
            skinny = b <= 2 and x_norm.dtype == torch.bfloat16 and self._wx.shape[0] <= 4096 <= self._wx.shape[1]
            ya = ops.gemv(x_norm, self._wx) if skinny else torch.nn.functional.linear(x_norm, self._wx)
            qa, kv_a, ik_raw = ya.split(
                [c.q_lora_rank, c.kv_lora_rank + c.qk_rope_head_dim, c.index_head_dim], dim=-1)
            c_q = self.q_a_layernorm(qa)
            # the c_q-side projection and the MLP's gate / up take the same kernel at one or two
            # tokens (252 against 255 us per layer of the 8-layer stack)
            wide = b <= 2 and c_q.dtype == torch.bfloat16
            q, iq_raw, w = (ops.gemv(c_q, self._wc) if wide else torch.nn.functional.linear(c_q, self._wc)).split(
                [h * (c.qk_nope_head_dim + c.qk_rope_head_dim), c.index_n_heads * c.index_head_dim, c.index_n_heads],
                dim=-1)
            # (rows of a batch must be dense for the fused prep launch; one row already is)
            q = (q if b == 1 else q.contiguous()).reshape(b, h, c.qk_nope_head_dim + c.qk_rope_head_dim)
            iq_raw = iq_raw.reshape(b, c.index_n_heads, c.index_head_dim)
        else:
            c_q = self.q_latent(x_norm)
            q = self.q_b_proj(c_q).view(b, h, c.qk_nope_head_dim + c.qk_rope_head_dim)
            kv_a = self.kv_a_proj(x_norm)
            iq_raw = self.index_q_proj(c_q).view(b, c.index_n_heads, c.index_head_dim)
            ik_raw = self.index_k_proj(x_norm)
            w = self.index_weights_proj(c_q)
        q_nope, q_rope = q.split([c.qk_nope_head_dim, c.qk_rope_head_dim], dim=-1)
        w_uk, _ = self._w_uk_uv()
        q_abs = torch.einsum("bhd,hdl->bhl", q_nope, w_uk)
        if cache.k_scale is not None and x_norm.dtype == torch.bfloat16:
            index_q = torch.empty(b, c.index_n_heads, c.index_head_dim, dtype=torch.uint8, device=x_norm.device)
            index_w = torch.empty(b, c.index_n_heads, dtype=torch.float32, device=x_norm.device)
            q_full = torch.empty(b, h, c.qk_head_dim, dtype=torch.bfloat16, device=x_norm.device)
            ops.decode_prep(iq_raw.contiguous(), w.contiguous(), ik_raw.contiguous(), kv_a.contiguous(),
                            q_abs.contiguous(), q_rope, self.kv_a_layernorm.weight, rope.mla_cos, rope.mla_sin,
                            rope.idx_cos, rope.idx_sin, positions, index_q, index_w, q_full, cache.index_k,
                            cache.k_scale, cache.kv, il, c.rms_norm_eps)
            return q_full, index_q, index_w
        q_rope = apply_rotary_at(q_rope, rope.mla_cos, rope.mla_sin, positions)
        c_kv, k_rope = kv_a.split([c.kv_lora_rank, c.qk_rope_head_dim], dim=-1)
        k_rope = apply_rotary_at(k_rope, rope.mla_cos, rope.mla_sin, positions)
        q_full = torch.cat([q_abs, q_rope], dim=-1)
        kv_row = torch.cat([self.kv_a_layernorm(c_kv), k_rope], dim=-1)
        cache.kv[batch_index, positions] = kv_row.to(cache.kv.dtype)
        iq = apply_rotary_at(iq_raw, rope.idx_cos, rope.idx_sin, positions, interleave=il)
        ik = apply_rotary_at(ik_raw, rope.idx_cos, rope.idx_sin, positions, interleave=il)
        if cache.k_scale is not None:
            ik8, sk = ops.quantize_e4m3_rowwise(ik.float().contiguous())
            cache.index_k[batch_index, positions] = ik8.view(torch.uint8)
            cache.k_scale[batch_index, positions] = sk
        else:
            cache.index_k[batch_index, positions] = ik.float()
        return q_full, iq, w

    def decode_indexer(self, iq, w, cache: LayerDecodeCache, seq_lens, pad_value: int = -1,
                       ws: Optional["IndexerWorkspace"] = None) -> torch.Tensor:
        """int32 [B, topk] selection over each sequence's first seq_lens keys. With
        a workspace the logits slab, the histogram, the top-k scratch and the
        result live in persistent buffers (nothing is allocated per step)."""
        topk = self.config.index_topk
        if cache.k_scale is not None:
            if iq.dtype == torch.uint8:  # already quantised by decode_project's fused launch
                iq8, wf = iq, w
            else:
                iq8, sq = ops.quantize_e4m3_rowwise(iq.float().contiguous())
                wf = (sq * w.float()).contiguous()
            if ws is None:
                logits = ops.indexer_scan_fp8(iq8, wf, cache.index_k, cache.k_scale, seq_lens)
                return ops.topk_select(logits, topk, seq_lens, pad_value=pad_value)
            logits = ops.indexer_scan_fp8(iq8, wf, cache.index_k, cache.k_scale, seq_lens, out=ws.logits, hist=ws.hist)
            return ops.topk_select(logits, topk, seq_lens, hist=ws.hist, pad_value=pad_value, out_idx=ws.indices,
                                   workspace=ws.topk_ws)
        logits = ops.indexer_scan_f32(iq.float().contiguous(), w.float().contiguous(), cache.index_k, seq_lens,
                                      out=None if ws is None else ws.logits)
        if ws is None:
            return ops.topk_select(logits, topk, seq_lens, pad_value=pad_value)
        return ops.topk_select(logits, topk, seq_lens, pad_value=pad_value, out_idx=ws.indices, workspace=ws.topk_ws)

    def decode_attention(self, q, cache: LayerDecodeCache, indices, seq_lens, beside_previous: bool = False) -> torch.Tensor:
        """Attention hidden output [B, hidden] of the new tokens; indices None = dense.
        ``beside_previous``: see :func:`ops.sparse_mla_decode` (used only when the queries need no
        conversion or padding launch in front of the attention)."""
        c = self.config
        if cache.k_scale is not None:
            h = q.shape[1]
            direct = q.dtype == torch.bfloat16 and h % ops.HEAD_BLOCK == 0 and q.is_contiguous()
            o = ops.sparse_mla_decode(_pad_heads(q.to(torch.bfloat16), ops.HEAD_BLOCK).contiguous(), cache.kv,
                                      indices, self.sm_scale, seq_lens,
                                      beside_previous=beside_previous and direct)[:, :h].to(q.dtype)
        else:
            o = ops.sparse_mla_f32(q.float().contiguous(), cache.kv, indices, c.kv_lora_rank, self.sm_scale,
                                   seq_lens).to(q.dtype)
        _, w_uv = self._w_uk_uv()
        ov = torch.einsum("bhl,hdl->bhd", o, w_uv)
        return self._reduced(self.o_proj(ov.reshape(ov.shape[0], c.num_attention_heads * c.v_head_dim)))
