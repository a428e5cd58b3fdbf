"""Decode-time driver of the hot path: persistent buffers, the three launches
(indexer scan -> top-k -> split-K sparse MLA) and CUDA-graph capture.

The reference's pure-PyTorch layer has no decode entry; its serving overlay
keeps per-shape persistent scratch and replays a captured graph
(sglang_overlay/mli-sglang-v0.5.16.patch:1274-1279, :1490-1505;
src/lagged_indexer_dsa/inference/modeling/fused_decode.py:46-119). This module
is that contract on top of the C ABI: every buffer is allocated once, lengths
are read on the device, and a step makes no allocation and no host sync.
"""

from __future__ import annotations

import ctypes
import dataclasses
import time
from typing import Optional

import torch

from . import ops


@dataclasses.dataclass
class LayerCache:
    """One layer's decode caches for ``n_seq`` sequences of capacity ``cap``.

    index_k ``[n_seq, cap, 128]`` e4m3 with k_scale ``[n_seq, cap]`` fp32, and
    the latent cache kv ``[n_seq, cap, 576]`` bf16 (or ``[n_seq, cap, 656]``
    uint8 fp8-packed rows)."""

    index_k: torch.Tensor
    k_scale: torch.Tensor
    kv: torch.Tensor

    @property
    def n_seq(self) -> int:
        return self.index_k.shape[0]

    @property
    def capacity(self) -> int:
        return self.index_k.shape[1]


class HotPathState:
    """Buffers of one decode step for ``rows`` query tokens (one per sequence).

    Inputs a caller fills before a step: ``index_q`` (e4m3 bytes), ``index_w``,
    ``q`` and ``seq_lens``. Outputs after a step: ``indices`` (the selection the
    indexer produced) and ``out`` (attention over ``attend`` indices)."""

    def __init__(self, rows: int, heads: int, index_heads: int, capacity: int, topk: int,
                 device, nsplit: Optional[int] = None, use_hist: bool = True) -> None:
        self.rows, self.heads, self.index_heads = rows, heads, index_heads
        self.capacity, self.topk = capacity, topk
        dev = torch.device(device)
        # The step's inputs live back to back in one allocation, and so do its
        # outputs, so a host-side caller moves each group with a single copy.
        nq, nw = rows * index_heads * ops.INDEX_DIM, rows * index_heads * 4
        nqq = rows * heads * ops.LATENT_DIM * 2
        self.in_arena = torch.zeros(nq + nw + nqq, dtype=torch.uint8, device=dev)
        self.index_q = self.in_arena[:nq].view(rows, index_heads, ops.INDEX_DIM)
        self.index_w = self.in_arena[nq:nq + nw].view(torch.float32).view(rows, index_heads)
        self.q = self.in_arena[nq + nw:].view(torch.bfloat16).view(rows, heads, ops.LATENT_DIM)
        self.seq_lens = torch.full((rows,), capacity, dtype=torch.int32, device=dev)
        slab = (capacity + 3) // 4 * 4
        self.logits = torch.empty(rows, slab, dtype=torch.float32, device=dev)
        # zero once; the select kernel re-zeroes it after every use
        self.hist = torch.zeros(rows, ops.HIST_BINS, dtype=torch.int32, device=dev) if use_hist else None
        no, ni = rows * heads * ops.VALUE_DIM * 2, rows * topk * 4
        self.out_arena = torch.zeros(no + ni, dtype=torch.uint8, device=dev)
        self.out = self.out_arena[:no].view(torch.bfloat16).view(rows, heads, ops.VALUE_DIM)
        self.indices = self.out_arena[no:].view(torch.int32).view(rows, topk)
        self.indices.fill_(-1)
        self.topk_ws = ops.topk_workspace(rows, capacity, dev)
        self.nsplit = nsplit or ops.default_nsplit(rows, heads, topk)
        self.scratch = ops.MlaScratch(rows, heads, self.nsplit, dev)

    # -- the three launches, on the current stream -----------------------------
    def run_indexer(self, cache: LayerCache, impl: int = 0) -> torch.Tensor:
        """Scan + select: fills and returns ``self.indices``."""
        logits = ops.indexer_scan_fp8(self.index_q, self.index_w, cache.index_k, cache.k_scale,
                                      self.seq_lens, ctx=self.capacity, out=self.logits,
                                      hist=self.hist, impl=impl)
        ops.topk_select(logits, self.topk, self.seq_lens, hist=self.hist, out_idx=self.indices,
                        workspace=self.topk_ws)
        return self.indices

    def run_attention(self, cache: LayerCache, attend: torch.Tensor, sm_scale: float,
                      beside_previous: bool = False) -> torch.Tensor:
        """Sparse MLA over ``attend`` (any ``[rows, topk]`` int32 selection). ``beside_previous``:
        ``attend`` and the queries do not come from the kernel enqueued just before (see
        :func:`ops.sparse_mla_decode`)."""
        return ops.sparse_mla_decode(self.q, cache.kv, attend, sm_scale, self.seq_lens,
                                     scratch=self.scratch, out=self.out, beside_previous=beside_previous)

    def run_lagged_chained(self, cache: LayerCache, attend: torch.Tensor, sm_scale: float) -> torch.Tensor:
        """Lagged order on ONE stream: this layer's scan and top-k, then the attention over
        ``attend`` (the previous layer's selection) enqueued behind the top-k and running beside
        it. One chain of programmatic dependents, no second stream and no join."""
        self.run_indexer(cache)
        return self.run_attention(cache, attend, sm_scale, beside_previous=True)

    def run_lagged_fused(self, cache: LayerCache, attend: torch.Tensor, sm_scale: float) -> torch.Tensor:
        """Lagged order in ONE role-split launch: attention over ``attend`` (the
        previous layer's selection) and this layer's indexer scan share the
        machine; the top-k then fills ``self.indices`` for the next layer."""
        ops.fused_decode(self.q, cache.kv, attend, sm_scale, self.index_q, self.index_w, cache.index_k,
                         cache.k_scale, self.seq_lens, scratch=self.scratch, out=self.out,
                         logits=self.logits, hist=self.hist)
        ops.topk_select(self.logits[:, :self.capacity], self.topk, self.seq_lens, hist=self.hist,
                        out_idx=self.indices, workspace=self.topk_ws)
        return self.out

    def run(self, cache: LayerCache, sm_scale: float, impl: int = 0) -> torch.Tensor:
        """Baseline order: the layer attends its own fresh selection."""
        self.run_indexer(cache, impl)
        return self.run_attention(cache, self.indices, sm_scale)

    def capture(self, cache: LayerCache, sm_scale: float, impl: int = 0) -> torch.cuda.CUDAGraph:
        """Captures ``run`` into a CUDA graph (after one eager warm-up launch)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.run(cache, sm_scale, impl)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.run(cache, sm_scale, impl)
        return graph


class HostDecoder:
    """End-to-end form with HOST buffers: copies a step's query operands from
    pinned host memory, replays the captured hot path and copies the attention
    output (and the selection) back. This is the call a host-side integrator
    makes when its tensors are not already on the device."""

    def __init__(self, state: HotPathState, cache: LayerCache, sm_scale: float, kernel_copies: bool = True,
                 poll: bool = True) -> None:
        self.state, self.cache = state, cache
        self.kernel_copies = kernel_copies
        self.poll = poll
        s = state
        # completion by polling: the graph's last node posts an epoch to pinned host memory
        self._epoch_dev = torch.zeros(1, dtype=torch.int32, device=s.in_arena.device)
        self._flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._flag_word = ctypes.c_uint32.from_address(self._flag.data_ptr())
        self._expected = 0
        # pinned mirrors of the two arenas, with the same views into them
        self.h_in = torch.zeros(s.in_arena.shape, dtype=torch.uint8).pin_memory()
        self.h_outbuf = torch.zeros(s.out_arena.shape, dtype=torch.uint8).pin_memory()
        nq, nw = s.index_q.numel(), s.index_w.numel() * 4
        no = s.out.numel() * 2
        self.h_index_q = self.h_in[:nq].view(s.index_q.shape)
        self.h_index_w = self.h_in[nq:nq + nw].view(torch.float32).view(s.index_w.shape)
        self.h_q = self.h_in[nq + nw:].view(torch.bfloat16).view(s.q.shape)
        self.h_out = self.h_outbuf[:no].view(torch.bfloat16).view(s.out.shape)
        self.h_indices = self.h_outbuf[no:].view(torch.int32).view(s.indices.shape)
        # One graph holds the whole step (input copy, kernels, selection copy), so a
        # step is a single launch on the host.
        self._side = torch.cuda.Stream()
        warm = torch.cuda.Stream()
        warm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(warm):
            self._body(sm_scale)
        torch.cuda.current_stream().wait_stream(warm)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._body(sm_scale)
        torch.cuda.synchronize()
        self._expected = int(self._flag.item())  # the warm-up launch above already posted once

    def _body(self, sm_scale: float) -> None:
        s = self.state
        main, side = torch.cuda.current_stream(), self._side
        # H2D in two pieces: index_q | index_w (8 KB, needed by the scan at once) in front of the
        # scan, q (needed only by the attention) while the indexer runs: by a kernel that copies
        # beside the top-k and completes after it, which keeps the whole step one chain of
        # programmatic dependents, or else by the copy engine on a forked stream joined before the
        # attention (a join gives the attention's node full dependencies).
        small = s.index_q.numel() + s.index_w.numel() * 4
        chained = self.kernel_copies and small % 16 == 0 and (self.h_in.numel() - small) % 16 == 0
        if chained:
            ops.copy_bytes(s.in_arena[:small], self.h_in[:small])  # a kernel node: starts sooner than a copy node
            s.run_indexer(self.cache)
            ops.copy_bytes(s.in_arena[small:], self.h_in[small:], beside_previous=True)
        else:
            side.wait_stream(main)
            s.in_arena[:small].copy_(self.h_in[:small], non_blocking=True)
            with torch.cuda.stream(side):
                s.in_arena[small:].copy_(self.h_in[small:], non_blocking=True)
            s.run_indexer(self.cache)
            main.wait_stream(side)
        # The attention's merge kernel writes its output straight into the pinned host buffer. The
        # selection (a few KB) goes back in the step's last node, which also posts the completion
        # word: one programmatic dependent of the merge kernel instead of a copy on the forked
        # stream, a join and a separate signal (a join gives its node full dependencies).
        sel_bytes = self.h_indices.numel() * 4
        fused_tail = self.poll and self.kernel_copies and sel_bytes % 16 == 0 and sel_bytes <= 1 << 20
        if not fused_tail:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                if self.kernel_copies:
                    ops.copy_bytes(self.h_indices, s.indices)
                else:
                    self.h_indices.copy_(s.indices, non_blocking=True)
        ops.sparse_mla_decode(s.q, self.cache.kv, s.indices, sm_scale, s.seq_lens, scratch=s.scratch,
                              out=self.h_out)
        if fused_tail:
            # (the selection was final three launches ago: it travels beside the merge kernel)
            ops.copy_post_epoch(self.h_indices, s.indices, self._epoch_dev, self._flag, beside_previous=True)
            return
        main.wait_stream(side)
        if self.poll:
            ops.post_epoch(self._epoch_dev, self._flag)  # after the join: every output is in host memory

    @property
    def h2d_bytes(self) -> int:
        return self.h_in.numel()

    @property
    def d2h_bytes(self) -> int:
        return self.h_outbuf.numel()

    def step(self) -> torch.Tensor:
        """Fill ``h_index_q``/``h_index_w``/``h_q`` first; returns ``h_out`` (and
        ``h_indices`` is valid) once the step has completed. With ``poll`` the host
        waits on the epoch word the graph's last node posts to pinned memory (falling
        back to a stream synchronise after 2 s) instead of a stream synchronise."""
        self.launch()
        return self.wait()

    def launch(self) -> None:
        """Enqueues the step and returns at once. A caller with several decoders (one per
        layer cache, each with its own pinned buffers) may launch the next one before it
        waits for this one, which hides the host's launch cost behind the device's work."""
        self.graph.replay()
        if self.poll:
            self._expected = (self._expected + 1) & 0xFFFFFFFF

    def wait(self) -> torch.Tensor:
        """Blocks until the step enqueued by the last :meth:`launch` has put its results into
        ``h_out`` / ``h_indices``."""
        if self.poll:
            word, want = self._flag_word, self._expected
            deadline = None
            spins = 0
            while word.value != want:
                spins += 1
                if spins & 0xFFFF == 0:
                    now = time.monotonic()
                    if deadline is None:
                        deadline = now + 2.0
                    elif now > deadline:
                        break
            if word.value != want:
                torch.cuda.current_stream().synchronize()
        else:
            torch.cuda.current_stream().synchronize()
        return self.h_out
