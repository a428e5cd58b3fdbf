"""Multi-GPU forms of the hot path on one NVLink/NVSwitch node, one process per GPU.

Two independent shardings:

* **Heads, tensor-parallel** (the reference's native scheme,
  src/lagged_indexer_dsa/inference/modeling/transformer.py:1323, :361-377):
  rank r owns MLA heads ``head_range(r)``; the latent cache, the index-key cache
  and the selection are replicated. The indexer is replicated too and is
  deterministic, so every rank selects the same set without the reference's
  rank-0 broadcast (transformer.py:1157-1164). The only collective is the
  all-reduce of the row-parallel output projection (``all_reduce_hidden``).
* **KV-sequence-sharded indexer** (not in the reference; its closest relative is
  the per-slice top-m + exact merge inside one GPU,
  kernels/cuda_fused_sparse_splitk.py:1914-2015): rank r scans keys
  ``key_range(r)``, keeps its local top-k as (global position, logit), one NCCL
  all-gather moves ``world * topk * 8`` bytes, and every rank merges the
  candidates with the same exact top-k kernel. The global top-k is a subset of
  the union of the local ones, and candidates arrive in ascending position
  order, so the merged set (ties to the lower position) equals the single-GPU
  selection bit for bit.

No kernel here reads a peer's memory: the gathered candidates land in local HBM
through NCCL before the merge kernel runs.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

SCAN_TILE = 128  # keys per scan tile: shard boundaries stay tile-aligned


def head_range(rank: int, world: int, heads: int) -> Tuple[int, int]:
    """Contiguous block of MLA heads owned by ``rank``."""
    if heads % world:
        raise ValueError(f"{heads} heads do not split over {world} ranks")
    per = heads // world
    return rank * per, (rank + 1) * per


def key_range(rank: int, world: int, n_keys: int, align: int = SCAN_TILE) -> Tuple[int, int]:
    """Contiguous KV range scanned by ``rank``: equal shares rounded up to
    ``align`` keys; trailing ranks may get a short or empty range."""
    per = -(-n_keys // world)
    per = -(-per // align) * align
    lo = min(rank * per, n_keys)
    return lo, min(lo + per, n_keys)


def interleave_gathered(gathered: torch.Tensor, world: int, rows: int, topk: int) -> torch.Tensor:
    """[world, rows, topk] (all-gather order) -> [rows, world * topk] with each
    row's candidates in rank order, i.e. ascending position order."""
    return gathered.reshape(world, rows, topk).permute(1, 0, 2).reshape(rows, world * topk).contiguous()


def all_reduce_hidden(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sums the per-rank partial outputs of a row-parallel projection in place."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, group=group)
    return x


class SeqShardedIndexer:
    """Indexer over a KV cache sharded by sequence range across ``group``.

    Each rank holds only its slice of the index keys (``local_ctx`` keys starting
    at global position ``key_lo``). ``select`` returns the global top-k
    positions, identical on every rank. Buffers are persistent: ``capture`` turns the
    call into two CUDA graphs with the one NCCL all-gather enqueued between them."""

    def __init__(self, rows: int, topk: int, local_ctx: int, key_lo: int, device,
                 group: Optional[dist.ProcessGroup] = None) -> None:
        from . import ops

        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rows, self.topk, self.local_ctx, self.key_lo = rows, topk, local_ctx, key_lo
        dev = torch.device(device)
        slab = (max(local_ctx, 1) + 3) // 4 * 4
        self.logits = torch.empty(rows, slab, dtype=torch.float32, device=dev)
        self.hist = torch.zeros(rows, ops.HIST_BINS, dtype=torch.int32, device=dev)
        self.local_ws = ops.topk_workspace(rows, max(local_ctx, 1), dev)
        # (index, logit) candidates travel as ONE buffer: [2, rows, topk] 32-bit words per rank
        self.cand = torch.empty(2, rows, topk, dtype=torch.int32, device=dev)
        self.cand_idx = self.cand[0]
        self.cand_val = self.cand[1].view(torch.float32)
        self.gath = torch.empty(self.world, 2, rows, topk, dtype=torch.int32, device=dev)
        self.merge_ws = ops.topk_workspace(rows, self.world * topk, dev)
        self.indices = torch.empty(rows, topk, dtype=torch.int32, device=dev)

    def select(self, index_q: torch.Tensor, index_w: torch.Tensor, index_k: torch.Tensor,
               k_scale: torch.Tensor, local_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """index_k / k_scale: this rank's slice ``[n_seq, local_ctx(, 128)]``;
        local_lens: visible keys inside the slice per row (None = all)."""
        self._local(index_q, index_w, index_k, k_scale, local_lens)
        if self.world == 1:
            self.indices.copy_(self.cand_idx)
            return self.indices
        self._exchange()
        self._merge()
        return self.indices

    def capture(self, index_q: torch.Tensor, index_w: torch.Tensor, index_k: torch.Tensor,
                k_scale: torch.Tensor, local_lens: Optional[torch.Tensor] = None,
                after: Optional[Callable[[torch.Tensor], None]] = None) -> Callable[[], torch.Tensor]:
        """``select`` on fixed buffers as two CUDA graphs around the one NCCL call: the
        local scan + top-k before it, the merge (and ``after(indices)``, e.g. this rank's
        attention over the merged set) behind it. The all-gather itself is enqueued
        between the two replays, outside any graph. Returns the step function."""
        self._local(index_q, index_w, index_k, k_scale, local_lens)  # warm-up, also of lazy state
        if self.world > 1:
            self._exchange()
            self._merge()
        else:
            self.indices.copy_(self.cand_idx)
        if after is not None:
            after(self.indices)
        torch.cuda.synchronize()
        g_local, g_merge = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_local):
            self._local(index_q, index_w, index_k, k_scale, local_lens)
        with torch.cuda.graph(g_merge):
            if self.world > 1:
                self._merge()
            else:
                self.indices.copy_(self.cand_idx)
            if after is not None:
                after(self.indices)

        def step() -> torch.Tensor:
            g_local.replay()
            if self.world > 1:
                self._exchange()
            g_merge.replay()
            return self.indices

        self._graphs = (g_local, g_merge)  # keep them alive with the indexer
        return step

    def _exchange(self) -> None:
        dist.all_gather_into_tensor(self.gath.view(-1), self.cand.view(-1), group=self.group)  # the one exchange step

    def _merge(self) -> None:
        idxs = interleave_gathered(self.gath[:, 0], self.world, self.rows, self.topk)
        vals = interleave_gathered(self.gath[:, 1], self.world, self.rows, self.topk).view(torch.float32)
        self.ops.topk_select(vals, self.topk, None, index_map=idxs, out_idx=self.indices, workspace=self.merge_ws)

    def _local(self, index_q: torch.Tensor, index_w: torch.Tensor, index_k: torch.Tensor,
               k_scale: torch.Tensor, local_lens: Optional[torch.Tensor]) -> None:
        ops = self.ops
        if self.local_ctx > 0:
            logits = ops.indexer_scan_fp8(index_q, index_w, index_k, k_scale, local_lens,
                                          ctx=self.local_ctx, out=self.logits, hist=self.hist)
            ops.topk_select(logits, self.topk, local_lens, hist=self.hist, out_idx=self.cand_idx,
                            out_val=self.cand_val, index_offset=self.key_lo, workspace=self.local_ws)
        else:  # an empty shard contributes only padding
            self.cand_idx.fill_(-1)
            self.cand_val.fill_(float("-inf"))
