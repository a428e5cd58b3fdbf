"""Multi-GPU forms of the hot path on one NVLink/NVSwitch node, one process per GPU.

Two independent shardings:

* **Heads, tensor-parallel** (the reference's native scheme,
  src/lagged_indexer_dsa/inference/modeling/transformer.py:1323, :361-377):
  rank r owns MLA heads ``head_range(r)``; the latent cache, the index-key cache
  and the selection are replicated. The indexer is replicated too and is
  deterministic, so every rank selects the same set without the reference's
  rank-0 broadcast (transformer.py:1157-1164). The only collective is the
  all-reduce of the row-parallel projections' partial outputs (``TensorParallel``).
* **KV-sequence-sharded indexer** (not in the reference; its closest relative is
  the per-slice top-m + exact merge inside one GPU,
  kernels/cuda_fused_sparse_splitk.py:1914-2015): rank r scans keys
  ``key_range(r)``, keeps its local top-k as (global position, logit), one exchange
  step moves ``world * topk * 8`` bytes (stores through peer-mapped pointers, or one
  NCCL all-gather), and every rank merges the candidates with the same exact top-k kernel. The global top-k is a subset of
  the union of the local ones, and candidates arrive in ascending position
  order, so the merged set (ties to the lower position) equals the single-GPU
  selection bit for bit.

No kernel here reads a peer's memory: candidates are stored into the peers' buffers (or
gathered by NCCL) and land in local HBM before the merge kernel reads them.
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


def tp_config(config, world: int):
    """The per-rank shapes of a layer that is tensor-parallel over ``world`` ranks: each rank owns
    ``num_attention_heads / world`` MLA heads and ``intermediate_size / world`` MLP columns
    (the reference's ColumnParallelLinear / RowParallelLinear split,
    src/lagged_indexer_dsa/inference/modeling/transformer.py:293-377, :1323). The indexer, the
    low-rank down-projections and the norms are replicated."""
    import dataclasses

    if config.num_attention_heads % world or config.intermediate_size % world:
        raise ValueError(f"{config.num_attention_heads} heads / {config.intermediate_size} MLP columns do not split "
                         f"over {world} ranks")
    return dataclasses.replace(config, num_attention_heads=config.num_attention_heads // world,
                               intermediate_size=config.intermediate_size // world)


def shard_state_dict(state: dict, config, rank: int, world: int) -> dict:
    """Rank ``rank``'s slice of a full model's ``state_dict``: rows of the column-parallel
    projections (q_b_proj and kv_b_proj per head, gate_proj / up_proj per MLP column), columns of
    the row-parallel ones (o_proj per head, down_proj per MLP column); everything else whole."""
    h0, h1 = head_range(rank, world, config.num_attention_heads)
    per_i = config.intermediate_size // world
    i0, i1 = rank * per_i, (rank + 1) * per_i
    dq = config.qk_nope_head_dim + config.qk_rope_head_dim
    dkv = config.qk_nope_head_dim + config.v_head_dim
    dv = config.v_head_dim
    out = {}
    for name, t in state.items():
        leaf = name.rsplit(".", 2)[-2] if name.endswith(".weight") else ""
        if leaf == "q_b_proj":
            t = t[h0 * dq:h1 * dq]
        elif leaf == "kv_b_proj":
            t = t[h0 * dkv:h1 * dkv]
        elif leaf == "o_proj":
            t = t[:, h0 * dv:h1 * dv]
        elif leaf in ("gate_proj", "up_proj"):
            t = t[i0:i1]
        elif leaf == "down_proj":
            t = t[:, i0:i1]
        out[name] = t.contiguous()
    return out


class TensorParallel:
    """The collective of a tensor-parallel layer: the sum of the row-parallel projections' partial
    outputs over the ranks (the reference's ``dist.all_reduce`` in RowParallelLinear,
    transformer.py:361-377). A decode activation (a few rows of ``hidden``) goes through
    ``ops.PeerAllReduce`` -- peer stores and a bounded wait, two small launches, capturable --
    larger tensors (prefill) through NCCL in fp32, as the reference does."""

    def __init__(self, hidden_size: int, device, group: Optional[dist.ProcessGroup] = None,
                 max_decode_rows: int = 4, wait_limit_s: float = 2.0, peers=None) -> None:
        from . import ops

        self.group = group
        if peers is not None:          # ranks emulated on one GPU: (PeerAllReduce of this rank, world, rank)
            self.ar, self.world, self.rank = peers
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
            self.ar = ops.PeerAllReduce(max_decode_rows * hidden_size, self.world, self.rank, device,
                                        wait_limit_s).connect(group)
        self.max_decode_elems = max_decode_rows * hidden_size

    def reduce(self, partial: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``partial`` over the ranks (plus ``residual``)."""
        if self.world == 1:
            return partial if residual is None else partial + residual
        if partial.dim() == 2 and partial.numel() <= self.max_decode_elems and partial.numel() % 4 == 0:
            return self.ar.all_reduce(partial.contiguous(), None if residual is None else residual.contiguous())
        y = partial.float()
        dist.all_reduce(y, group=self.group)
        y = y.to(partial.dtype)
        return y if residual is None else y + residual


class SeqShardedIndexer:
    """Indexer over a KV cache sharded by sequence range across ``group``.

    Each rank holds only its slice of the index keys (``local_ctx`` keys starting at global
    position ``key_lo``). ``select`` returns the global top-k positions, identical on every
    rank and equal to the single-GPU selection bit for bit. Two ways to move the candidates:

    * ``exchange="p2p"`` (default): the local top-k stores its (position, logit) pairs straight
      into every rank's gather buffers through peer-mapped pointers and posts a flag; the merge
      kernel waits for the flags on the device, with a limit (``ops.CandidateExchange``). A step
      is kernels in stream order, so it can be captured in ONE CUDA graph together with the
      attention behind it.
    * ``exchange="nccl"``: local top-k, one ``all_gather_into_tensor`` of the packed candidates,
      merge. ``capture`` then makes two graphs with the eager NCCL call between the replays."""

    def __init__(self, rows: int, topk: int, local_ctx: int, key_lo: int, device,
                 group: Optional[dist.ProcessGroup] = None, exchange: str = "p2p",
                 wait_limit_s: float = 2.0) -> None:
        from . import ops

        if exchange not in ("p2p", "nccl"):
            raise ValueError("exchange must be 'p2p' or 'nccl'")
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows, self.topk, self.local_ctx, self.key_lo = rows, topk, local_ctx, key_lo
        self.exchange = exchange
        dev = torch.device(device)
        slab = (max(local_ctx, 1) + 3) // 4 * 4
        self.logits = torch.empty(rows, slab, dtype=torch.float32, device=dev)
        self.hist = torch.zeros(rows, ops.HIST_BINS, dtype=torch.int32, device=dev)
        self.local_ws = ops.topk_workspace(rows, max(local_ctx, 1), dev)
        self.indices = torch.empty(rows, topk, dtype=torch.int32, device=dev)
        self.xchg = None
        if exchange == "p2p":
            self.xchg = ops.CandidateExchange(rows, topk, self.world, self.rank, dev, wait_limit_s).connect(group)
            if local_ctx <= 0:  # an empty shard pushes a row of -inf: every entry comes out as padding
                self._empty = torch.full((rows, 4), float("-inf"), dtype=torch.float32, device=dev)
        else:
            # (index, logit) candidates travel as ONE buffer: [2, rows, topk] 32-bit words per rank
            self.cand = torch.empty(2, rows, topk, dtype=torch.int32, device=dev)
            self.cand_idx = self.cand[0]
            self.cand_val = self.cand[1].view(torch.float32)
            self.gath = torch.empty(self.world, 2, rows, topk, dtype=torch.int32, device=dev)
            self.merge_ws = ops.topk_workspace(rows, self.world * topk, dev)

    def select(self, index_q: torch.Tensor, index_w: torch.Tensor, index_k: torch.Tensor,
               k_scale: torch.Tensor, local_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """index_k / k_scale: this rank's slice ``[n_seq, local_ctx(, 128)]``;
        local_lens: visible keys inside the slice per row (None = all)."""
        self._local(index_q, index_w, index_k, k_scale, local_lens)
        if self.exchange == "p2p":
            return self.xchg.merge(self.indices)
        if self.world == 1:
            self.indices.copy_(self.cand_idx)
            return self.indices
        self._exchange()
        self._merge()
        return self.indices

    def capture(self, index_q: torch.Tensor, index_w: torch.Tensor, index_k: torch.Tensor,
                k_scale: torch.Tensor, local_lens: Optional[torch.Tensor] = None,
                after: Optional[Callable[[torch.Tensor], None]] = None) -> Callable[[], torch.Tensor]:
        """``select`` (and ``after(indices)``, e.g. this rank's attention over the merged set) on
        fixed buffers as CUDA graphs. With the p2p exchange that is ONE graph. With NCCL it is two
        graphs around the one all-gather, which is enqueued between the two replays, outside any
        graph. Every rank must call it (the warm-up runs one real step). Returns the step function."""
        args = (index_q, index_w, index_k, k_scale, local_lens)
        self.select(*args)  # warm-up, also of lazy state
        if after is not None:
            after(self.indices)
        torch.cuda.synchronize()
        if self.exchange == "p2p":
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.select(*args)
                if after is not None:
                    after(self.indices)
            self._graphs = (graph,)

            def step() -> torch.Tensor:
                graph.replay()
                return self.indices

            return step
        g_local, g_merge = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_local):
            self._local(*args)
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
            if self.exchange == "p2p":
                self.xchg.push(logits, local_lens, hist=self.hist, index_offset=self.key_lo)
            else:
                ops.topk_select(logits, self.topk, local_lens, hist=self.hist, out_idx=self.cand_idx,
                                out_val=self.cand_val, index_offset=self.key_lo, workspace=self.local_ws)
        elif self.exchange == "p2p":
            self.xchg.push(self._empty)
        else:  # an empty shard contributes only padding
            self.cand_idx.fill_(-1)
            self.cand_val.fill_(float("-inf"))
