"""A stack of DSA blocks under the three schedules, full-sequence and decode.

``DSAModel.forward`` keeps the reference's signature and control flow
(src/lagged_indexer_dsa/model.py:73-144): BASELINE attends the layer's own
selection; the lagged modes attend the previous layer's, with layer 0 cold
started, and a layer runs an indexer only if a later layer consumes it.

The decode half has no counterpart in the reference's pure-PyTorch model; it is
the GPU realisation of what the serving overlay does to SGLang
(sglang_overlay/mli-sglang-v0.5.16.patch:2942-2997 fork, :1820-1832 and
:3858-3870 join, :4516-4532 drain, :1785-1802 pre-created stream): in the lagged
modes layer l's indexer (quantise -> FP8 scan -> top-k) is launched on a second
CUDA stream and joined just before layer l+1's attention, so it overlaps layer
l's attention, output projection and MLP; the whole step is capturable in one
CUDA graph. ``retention`` keeps indexers on a subset of layers ("F") and lets
the others ("S") reuse the carried selection (overlay :33-51, :4027-4049).
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn

from .config import AttentionType, ColdStartPolicy, DSAConfig, ScheduleMode
from .dsa_layer import DSALayer, IndexerWorkspace, LayerDecodeCache, RMSNorm, RopeCaches
from .rope import build_rope_cache


@dataclasses.dataclass
class ForwardTrace:
    """Per-layer record of a forward pass (reference model.py:23-33)."""

    final_hidden: torch.Tensor
    indices_used: List[Optional[torch.Tensor]]
    indices_produced: List[Optional[torch.Tensor]]


def lagged_producers(types: Sequence[AttentionType]) -> List[bool]:
    """Layer L runs an indexer under the lag iff layer L+1 is a DSA layer
    (reference model.py:61-71)."""
    n = len(types)
    return [(i + 1 < n and types[i + 1] is AttentionType.DSA) for i in range(n)]


def parse_retention(pattern: Optional[str], n_layers: int) -> List[bool]:
    """'F'/'S' per layer -> runs-an-indexer flags. None keeps every indexer; an
    integer string 'k' keeps every k-th. Layer 0 always runs one (overlay :37-44)."""
    if pattern is None:
        return [True] * n_layers
    if pattern.isdigit():
        k = max(1, int(pattern))
        flags = [(i % k) == 0 for i in range(n_layers)]
    else:
        if len(pattern) != n_layers or set(pattern) - {"F", "S"}:
            raise ValueError(f"retention pattern must be {n_layers} characters of F/S, got {pattern!r}")
        flags = [ch == "F" for ch in pattern]
    flags[0] = True
    return flags


@dataclasses.dataclass
class DecodeState:
    """Mutable decode state: per-layer caches, device-side lengths, rotary tables,
    the side stream of the lagged schedule and the selection being carried."""

    caches: List[LayerDecodeCache]
    rope: RopeCaches
    positions: torch.Tensor      # int64 [B]: position of the NEXT token
    seq_lens: torch.Tensor       # int32 [B]: keys visible to the next token (= positions + 1 once appended)
    batch_index: torch.Tensor    # int64 [B]
    side_stream: torch.cuda.Stream
    runs_indexer: List[bool]
    fp8: bool
    workspaces: List[IndexerWorkspace] = dataclasses.field(default_factory=list)
    carried: Optional[torch.Tensor] = None


class DSAModel(nn.Module):
    def __init__(self, config: DSAConfig) -> None:
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([DSALayer(config) for _ in range(config.num_hidden_layers)])
        self.final_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    # ------------------------------------------------------------------ tensor parallelism
    @classmethod
    def tensor_parallel(cls, full_config: DSAConfig, full_state: dict, device, dtype=None, group=None,
                        peers=None) -> "DSAModel":
        """This rank's part of a model that is tensor-parallel over the process group: MLA heads
        and MLP columns are split (``parallel.tp_config`` / ``shard_state_dict``), the indexer,
        the low-rank down-projections and the norms are replicated, and every layer sums the
        partial outputs of its row-parallel ``o_proj`` / ``down_proj`` over the ranks
        (``parallel.TensorParallel``; the reference's RowParallelLinear,
        src/lagged_indexer_dsa/inference/modeling/transformer.py:361-377). The indexer is
        deterministic, so every rank selects the same keys without the reference's rank-0
        broadcast (:1157-1164). ``full_state`` is the state_dict of the unsharded model (every
        rank passes the same one); None leaves this rank's shard at its random initialisation,
        created on ``device`` (benchmarks with random weights: no rank ever holds the full model).
        ``peers`` = (PeerAllReduce, world, rank) emulates the ranks on one GPU."""
        from .parallel import TensorParallel, shard_state_dict, tp_config
        import torch.distributed as dist

        if peers is not None:
            _, world, rank = peers
        else:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        if full_state is None:
            with torch.device(device):
                model = cls(tp_config(full_config, world))
        else:
            model = cls(tp_config(full_config, world))
            model.load_state_dict(shard_state_dict(full_state, full_config, rank, world))
        model = model.to(device=device, dtype=dtype).eval()
        tp = TensorParallel(full_config.hidden_size, device, group, peers=peers)
        for layer in model.layers:
            layer.tp = tp  # the layers run one after the other: one set of buffers serves them all
        model.tp = tp
        return model

    # ------------------------------------------------------------------ shared helpers
    def _build_rope(self, seq_len: int, device, dtype) -> RopeCaches:
        c = self.config
        mc, ms = build_rope_cache(seq_len, c.qk_rope_head_dim, c.rope_theta, device, dtype)
        ic, is_ = build_rope_cache(seq_len, c.index_head_dim, c.rope_theta, device, dtype,
                                   interleave=c.indexer_rope_interleave)
        return RopeCaches(mc, ms, ic, is_)

    def _cold_start_indices(self, layer: DSALayer, x_norm, rope, cold_start: ColdStartPolicy):
        if cold_start is ColdStartPolicy.DENSE:
            return None
        if cold_start is ColdStartPolicy.EAGER:
            return layer.indexer_indices(x_norm, rope)
        raise ValueError(f"unknown cold start policy: {cold_start}")

    def _lagged_indexer_layers(self, types) -> List[bool]:
        return lagged_producers(types)

    # ------------------------------------------------------------------ reference API
    def forward(self, inputs_embeds: torch.Tensor, mode: ScheduleMode,
                cold_start: ColdStartPolicy = ColdStartPolicy.DENSE, record: bool = False):
        if inputs_embeds.dim() != 3:
            raise ValueError(f"inputs_embeds must be [B,S,H], got {tuple(inputs_embeds.shape)}")
        if not inputs_embeds.is_cuda:
            raise RuntimeError("this implementation runs on a CUDA device only (there is no CPU path)")
        rope = self._build_rope(inputs_embeds.shape[1], inputs_embeds.device, inputs_embeds.dtype)
        types = self.config.resolved_attention_types
        produces = lagged_producers(types)
        x = inputs_embeds
        prev: Optional[torch.Tensor] = None
        used, produced = [], []
        for li, layer in enumerate(self.layers):
            x_norm = layer.attn_norm(x)
            is_dsa = types[li] is AttentionType.DSA
            if mode is ScheduleMode.BASELINE:
                made = layer.indexer_indices(x_norm, rope) if is_dsa else None
                attend = made
                attn = layer.attention_output(x_norm, rope, attend)
            elif mode in (ScheduleMode.LAGGED_REFERENCE, ScheduleMode.LAGGED_FUSED):
                if not is_dsa:
                    attend = None
                elif li == 0:
                    attend = self._cold_start_indices(layer, x_norm, rope, cold_start)
                else:
                    attend = prev
                if mode is ScheduleMode.LAGGED_REFERENCE:
                    attn = layer.attention_output(x_norm, rope, attend)
                    made = layer.indexer_indices(x_norm, rope) if produces[li] else None
                else:
                    attn, made = layer.fused_attention_and_indices(x_norm, rope, attend,
                                                                   produce_indexer=produces[li])
            else:
                raise ValueError(f"unknown schedule mode: {mode}")
            h = x + attn
            x = h + layer.mlp(layer.ffn_norm(h))
            prev = made
            if record:
                used.append(attend)
                produced.append(made)
        x = self.final_norm(x)
        return ForwardTrace(x, used, produced) if record else x

    # ------------------------------------------------------------------ decode
    def init_decode(self, batch: int, capacity: int, fp8: Optional[bool] = None,
                    retention: Optional[str] = None) -> DecodeState:
        """Allocates the caches for ``batch`` sequences of up to ``capacity`` tokens.
        fp8=True stores e4m3 index keys + bf16 latent rows (needs the production
        geometry); fp8=False stores fp32 caches of any width."""
        p = next(self.parameters())
        if not p.is_cuda:
            raise RuntimeError("decode needs the model on a CUDA device")
        if fp8 is None:
            fp8 = self.config.is_production_geometry and p.dtype == torch.bfloat16
        if fp8 and not self.config.is_production_geometry:
            raise ValueError("fp8 caches need the production geometry (576-wide latent, 128-wide index keys)")
        dev = p.device
        if fp8 and p.dtype == torch.bfloat16:
            for layer in self.layers:  # two stacked GEMVs per layer instead of six small ones
                if not layer._stacked():
                    layer.fuse_decode_weights()
        caches = [layer.new_cache(batch, capacity, dev, fp8) for layer in self.layers]
        return DecodeState(
            caches=caches, rope=self._build_rope(capacity, dev, p.dtype),
            positions=torch.zeros(batch, dtype=torch.int64, device=dev),
            seq_lens=torch.zeros(batch, dtype=torch.int32, device=dev),
            batch_index=torch.arange(batch, device=dev),
            # (default priority: a high-priority stream, the reference's HH_LAG_STREAM_PRIORITY,
            # sglang_overlay/mli-sglang-v0.5.16.patch:1795-1800, shortens the bare attention + indexer
            # pair by 2 us but measured 0.5 us per layer slower inside the full stack, where the
            # main stream's projections and all-reduces are the critical path)
            side_stream=torch.cuda.Stream(device=dev),
            runs_indexer=parse_retention(retention, len(self.layers)), fp8=fp8,
            workspaces=[IndexerWorkspace.create(batch, capacity, self.config.index_topk, dev, fp8)
                        for _ in self.layers])

    @torch.no_grad()
    def prefill(self, state: DecodeState, inputs_embeds: torch.Tensor,
                mode: ScheduleMode = ScheduleMode.BASELINE,
                cold_start: ColdStartPolicy = ColdStartPolicy.DENSE) -> torch.Tensor:
        """Runs the full-sequence forward over a prompt [B,S,hidden], filling every
        layer's caches on the way; returns the final hidden states."""
        b, s, _ = inputs_embeds.shape
        rope = RopeCaches(state.rope.mla_cos[:s], state.rope.mla_sin[:s], state.rope.idx_cos[:s], state.rope.idx_sin[:s])
        types = self.config.resolved_attention_types
        produces = lagged_producers(types)
        x, prev = inputs_embeds, None
        for li, layer in enumerate(self.layers):
            x_norm = layer.attn_norm(x)
            layer.fill_cache(state.caches[li], x_norm, rope)
            is_dsa = types[li] is AttentionType.DSA
            if mode is ScheduleMode.BASELINE:
                made = layer.indexer_indices(x_norm, rope) if is_dsa else None
                attend = made
            else:
                attend = (None if not is_dsa else
                          self._cold_start_indices(layer, x_norm, rope, cold_start) if li == 0 else prev)
                made = layer.indexer_indices(x_norm, rope) if produces[li] else None
            h = x + layer.attention_output(x_norm, rope, attend)
            x = h + layer.mlp(layer.ffn_norm(h))
            prev = made
        state.positions.fill_(s)
        state.seq_lens.fill_(s)
        return self.final_norm(x)

    @torch.no_grad()
    def decode_step(self, state: DecodeState, x: torch.Tensor, mode: ScheduleMode,
                    cold_start: ColdStartPolicy = ColdStartPolicy.DENSE, overlap=True,
                    record: Optional[dict] = None, lag_depth: int = 1) -> torch.Tensor:
        """One new token per sequence: x [B,hidden] -> final hidden [B,hidden].

        Appends the token's keys to every layer's caches at ``state.positions``
        and advances the device-side lengths. In the lagged modes with
        ``overlap`` the indexers run on ``state.side_stream``; with ``overlap="chained"``
        they stay on the current stream and the attention, which reads the PREVIOUS
        layer's selection, is enqueued behind the layer's scan and top-k and runs beside
        the top-k (one chain of programmatic dependents, no second stream). ``lag_depth`` k >= 2
        lets an indexer overlap k refresh spans instead of one (see
        ``_decode_step_depth``). Capturable in a CUDA graph (no host sync, lengths
        stay on the device)."""
        if lag_depth < 1:
            raise ValueError("lag_depth must be >= 1")
        chained = overlap == "chained"
        if lag_depth > 1:
            if mode is ScheduleMode.BASELINE:
                raise ValueError("lag_depth > 1 needs a lagged schedule mode")
            if chained:
                raise ValueError("the chained overlap is defined for lag_depth 1")
            return self._decode_step_depth(state, x, cold_start, overlap, record, lag_depth)
        types = self.config.resolved_attention_types
        n = len(self.layers)
        lagged = mode is not ScheduleMode.BASELINE
        main = torch.cuda.current_stream()
        side = state.side_stream if (lagged and overlap is True) else None
        state.seq_lens.add_(1)  # the new token sees itself
        carried: Optional[torch.Tensor] = None
        pending = False  # an indexer is in flight on the side stream
        used, produced = [], []
        x_norm = self.layers[0].attn_norm(x)
        for li, layer in enumerate(self.layers):
            cache = state.caches[li]
            is_dsa = types[li] is AttentionType.DSA
            q, iq, w = layer.decode_project(x_norm, state.rope, state.positions, cache, state.batch_index)
            made = None
            beside = False
            if not lagged:
                if is_dsa and state.runs_indexer[li]:
                    carried = made = layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                attend = carried if is_dsa else None
            else:
                if pending:  # join layer li-1's indexer before its selection is read
                    main.wait_stream(side)
                    pending = False
                if not is_dsa:
                    attend = None
                elif li == 0:
                    attend = (None if cold_start is ColdStartPolicy.DENSE
                              else layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li]))
                else:
                    attend = carried
                # a layer produces iff it keeps its indexer and the next layer attends sparsely
                if state.runs_indexer[li] and li + 1 < n and types[li + 1] is AttentionType.DSA:
                    if side is not None:
                        side.wait_stream(main)  # fork: needs iq, w and the appended key
                        with torch.cuda.stream(side):
                            made = layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                        pending = True
                    else:
                        made = layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                        # The attention may run beside the two launches just enqueued when nothing it
                        # reads comes from them: the selection is an earlier layer's (li > 0), and the
                        # indexer call allocated nothing that the attention's scratch could reuse.
                        beside = (chained and li > 0 and attend is not None and cache.k_scale is not None
                                  and iq.dtype == torch.uint8 and state.workspaces[li] is not None)
            attn = layer.decode_attention(q, cache, attend, state.seq_lens, beside_previous=beside)
            x, x_norm = self._residual_tail(li, x, attn)
            if lagged and made is not None:
                carried = made  # becomes visible to layer li+1 after the join
            if record is not None:
                used.append(attend)
                produced.append(made)
        if pending:  # never leave a fork dangling (a captured graph must end joined)
            main.wait_stream(side)
        state.positions.add_(1)
        state.carried = carried
        if record is not None:
            record["used"], record["produced"] = used, produced
        return x_norm  # the last layer's tail applied the final norm

    def _residual_tail(self, li: int, x: torch.Tensor, attn: torch.Tensor):
        """``h = x + attn; x' = h + mlp(ffn_norm(h))`` and the norm the next consumer
        applies to ``x'`` (the next layer's attn_norm, or the final norm after the last
        layer): each residual addition is fused with the norm that follows it."""
        layer = self.layers[li]
        h, h_norm = layer.ffn_norm.add_forward(x, attn)
        nxt = self.layers[li + 1].attn_norm if li + 1 < len(self.layers) else self.final_norm
        return nxt.add_forward(h, layer.mlp(h_norm))

    def _decode_step_depth(self, state: DecodeState, x: torch.Tensor, cold_start: ColdStartPolicy,
                           overlap: bool, record: Optional[dict], depth: int) -> torch.Tensor:
        """Lag depth k >= 2 (overlay ``_hh_lag_refresh_dispatch_depth``,
        sglang_overlay/mli-sglang-v0.5.16.patch:3017-3100): a refresh layer (one that
        keeps its indexer) launches its indexer on the side stream, records an
        event and queues the fresh set in a FIFO of depth k; once the FIFO is
        full the layer pops the OLDEST entry, joins on that entry's event only
        and attends it, so an indexer overlaps k refresh spans. While the FIFO
        fills, the layer attends the incoming carry. The carry-out of a refresh
        layer is the set it ATTENDED, which the skip layers after it copy. The
        first sparse layer bootstraps: EAGER runs its indexer serially and
        attends it (nothing queued); DENSE attends densely and queues its set."""
        types = self.config.resolved_attention_types
        main = torch.cuda.current_stream()
        side = state.side_stream if overlap else None
        state.seq_lens.add_(1)  # the new token sees itself
        carried: Optional[torch.Tensor] = None
        fifo: List[Tuple[Optional[torch.cuda.Event], torch.Tensor]] = []
        booted = False
        forked = False
        used, produced = [], []
        x_norm = self.layers[0].attn_norm(x)
        for li, layer in enumerate(self.layers):
            cache = state.caches[li]
            is_dsa = types[li] is AttentionType.DSA
            q, iq, w = layer.decode_project(x_norm, state.rope, state.positions, cache, state.batch_index)
            made = None

            def dispatch():
                """This layer's indexer, deferred: (event, fresh set)."""
                nonlocal forked
                if side is None:
                    return None, layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                side.wait_stream(main)  # fork: needs iq, w and the appended key
                with torch.cuda.stream(side):
                    fresh = layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                    done = torch.cuda.Event()
                    done.record(side)
                forked = True
                return done, fresh

            if not is_dsa:
                attend = None
            elif not booted:
                booted = True
                if cold_start is ColdStartPolicy.DENSE:
                    attend = None
                    if state.runs_indexer[li]:
                        ev, made = dispatch()
                        fifo.append((ev, made))
                else:
                    attend = made = layer.decode_indexer(iq, w, cache, state.seq_lens, ws=state.workspaces[li])
                carried = attend
            elif state.runs_indexer[li]:
                ev, made = dispatch()
                if len(fifo) >= depth:
                    old_ev, attend = fifo.pop(0)
                    if old_ev is not None:
                        main.wait_event(old_ev)  # join on the oldest entry only
                else:
                    attend = carried  # pipeline fill
                fifo.append((ev, made))
                carried = attend
            else:
                attend = carried
            attn = layer.decode_attention(q, cache, attend, state.seq_lens)
            x, x_norm = self._residual_tail(li, x, attn)
            if record is not None:
                used.append(attend)
                produced.append(made)
        if forked:  # drain: never leave a fork dangling (a captured graph must end joined)
            main.wait_stream(side)
        state.positions.add_(1)
        state.carried = carried
        if record is not None:
            record["used"], record["produced"] = used, produced
        return x_norm  # the last layer's tail applied the final norm

    def capture_decode(self, state: DecodeState, mode: ScheduleMode,
                       cold_start: ColdStartPolicy = ColdStartPolicy.DENSE, overlap=True,
                       lag_depth: int = 1):
        """Captures one decode step in a CUDA graph. Returns (graph, x_in, x_out):
        copy the token's hidden state into x_in, replay, read x_out. The caches
        and lengths advance on every replay exactly as in eager mode. Warm-up
        steps run first on a scratch copy of the lengths so the state is left
        where it was."""
        p = next(self.parameters())
        b = state.positions.shape[0]
        x_in = torch.zeros(b, self.config.hidden_size, dtype=p.dtype, device=p.device)
        saved = (state.positions.clone(), state.seq_lens.clone())
        warm = torch.cuda.Stream(device=p.device)
        warm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(warm):
            for _ in range(2):
                self.decode_step(state, x_in, mode, cold_start, overlap, lag_depth=lag_depth)
                state.positions.copy_(saved[0])
                state.seq_lens.copy_(saved[1])
        torch.cuda.current_stream().wait_stream(warm)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            x_out = self.decode_step(state, x_in, mode, cold_start, overlap, lag_depth=lag_depth)
        # the capture itself does not execute: lengths are still at their saved values
        return graph, x_in, x_out
