"""Benchmark of the DSA decode hot path (indexer scan -> top-2048 -> split-K
sparse MLA) at the DeepSeek-V3.2 single-layer decode shape: batch 1, context
131072, FP8 index keys, 128 MLA heads over a bf16 latent cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one layer's hot path for one decode token. Steps cycle over
`--layers` distinct per-layer caches so a step never finds its keys in L2.
Prints ONE JSON line (rank 0). With --impl reference the CPU oracle (a port of
the reference's PyTorch path) is timed on the host cores instead.

Under torchrun (N > 1) MLA heads are split tensor-parallel across ranks and the
two forms are timed and the faster one is the line's value: the indexer
replicated, as the reference does under TP
(src/lagged_indexer_dsa/inference/modeling/transformer.py:673-677, :1323), and
the scan split by KV range with the per-rank top-2048 candidates exchanged by
peer stores inside the step's graph and merged. Before the timed region the
N-rank result is checked against the one-GPU result on the same inputs.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

CTX = 131072
HEADS = 128
INDEX_HEADS = 64
TOPK = 2048
SM_SCALE = 192 ** -0.5
SCAN_BYTES_PER_KEY = 132          # 128 B e4m3 key + 4 B fp32 scale
SCAN_TRAFFIC_CTX128K = 17368576   # bytes: ncu dram read + write of one scan launch over 131072 keys
METRIC = "dsa_decode_layer_tokens_per_s_ctx128k"
UNIT = "tok/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--layers", type=int, default=16, help="distinct per-layer caches cycled through")
    ap.add_argument("--graph-per-layer", action="store_true",
                    help="one CUDA graph per step instead of one graph over --layers consecutive steps")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scan-impl", type=int, default=0, help="0 tcgen05, 1 legacy mma.sync")
    ap.add_argument("--workload", default="layer_decode", choices=["layer_decode", "batch32_paged", "mli_stack"],
                    help="layer_decode = BASELINE config 2 (the default bench line); the others are extra measurements")
    return ap.parse_args()


def workload_config(args, world):
    return {
        "workload": "deepseek_v3.2_single_layer_decode (BASELINE config 2)",
        "batch": 1, "context": args.ctx, "index_heads": INDEX_HEADS, "index_dim": 128,
        "index_key_dtype": "e4m3+fp32 scale", "topk": TOPK, "mla_heads": HEADS, "latent_dim": 576,
        "latent_dtype": "bf16", "sm_scale": "1/sqrt(192)",
        "parallelism": "tp%d_heads" % world if world == 1 else "tp%d_heads: the faster of +replicated_indexer and +seq_sharded_indexer" % world,
        "l2": "%d distinct per-layer caches cycled (%.0f MB of index keys + %.0f MB of latent rows): "
              "inputs larger than the 126 MB L2" % (args.layers, args.layers * args.ctx * 132 / 1e6,
                                                    args.layers * args.ctx * 1152 / 1e6),
        "launch": ("one CUDA graph per layer step (4 kernels: scan, top-k, attention partials, combine)"
                   if args.graph_per_layer or args.layers <= 1 else
                   "one CUDA graph over %d consecutive layer steps, as a model's decode step is captured "
                   "(4 kernels per step: scan, top-k, attention partials, combine; 5 with the sequence-sharded "
                   "indexer: scan, local top-k + peer stores, merge, partials, combine); "
                   "steps beyond a multiple of %d share one more graph" % (args.layers, args.layers)),
    }


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ CPU arm
# The reference's own CPU code for this path is three host functions of its kernel file:
# ref_indexer_logits_fp8 (kernels/cuda_fused_sparse_splitk.py:2990-2992), torch.topk on the
# logits (src/lagged_indexer_dsa/inference/modeling/transformer.py:1156) and ref_sparse_mla
# (kernels/cuda_fused_sparse_splitk.py:2950-2966). Where oracle/_ref holds a copy of the
# reference (built by oracle/build_ref.py on a machine that has the checkout) those functions
# are imported from it and timed: kind "reference". Otherwise the oracle's restatement of the
# same functions is timed: kind "port".
REF_MAX_STEPS = 2048  # cap on warm-up + timed steps of the CPU arm (two to three minutes at 60-80 ms per step)


def cpu_step_inputs(ctx, seed=0):
    from oracle import dsa_oracle as O

    g = torch.Generator().manual_seed(seed)
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(torch.randn(1, INDEX_HEADS, 128, generator=g),
                                                 torch.randn(ctx, 128, generator=g),
                                                 torch.randn(1, INDEX_HEADS, generator=g) / 8)
    q = torch.randn(1, HEADS, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(ctx, 576, generator=g).to(torch.bfloat16)
    return iq8, ik8, wp, sk, q, kv


def cpu_step_fn(ctx):
    """Returns (step(inputs), kind): the reference's own functions when oracle/_ref has them."""
    from oracle import build_ref
    from oracle import dsa_oracle as O

    ref = build_ref.load_ref()
    if ref is not None:
        def step(inputs):
            iq8, ik8, wp, sk, q, kv = inputs
            logits = ref.ref_indexer_logits_fp8(iq8[0:1], ik8, wp, sk)                  # [1, ctx]
            idx = torch.topk(logits, TOPK, dim=-1).indices.to(torch.int32)               # [1, topk]
            return ref.ref_sparse_mla(q.unsqueeze(0), kv.view(1, ctx, 1, 576), idx, SM_SCALE, "cpu")

        return step, "reference"

    def step(inputs):
        iq8, ik8, wp, sk, q, kv = inputs
        logits = O.indexer_logits_fp8(iq8, ik8, wp, sk, chunk=32768)
        idx = torch.topk(logits, TOPK, dim=-1).indices
        return O.sparse_mla_decode(q, kv, idx, [ctx], SM_SCALE)

    return step, "port"


def time_cpu(ctx, steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inputs = cpu_step_inputs(ctx)
    step, kind = cpu_step_fn(ctx)
    for _ in range(warmup):
        step(inputs)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(inputs)
    dt = (time.perf_counter() - t0) / steps
    return dt, cores, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    warmup = max(3, args.warmup)  # (the GPU arm never runs fewer than three warm-ups either)
    steps = max(1, args.steps)
    capped = ""
    if warmup + steps > REF_MAX_STEPS:  # honour the arguments up to the cap, and say so
        warmup = min(warmup, 64)
        steps = REF_MAX_STEPS - warmup
        capped = f" (capped at {REF_MAX_STEPS} steps in total: asked for --steps {args.steps} --warmup {args.warmup})"
    dt, cores, kind = time_cpu(args.ctx, steps, warmup)
    val = 1.0 / dt
    what = ("the reference's ref_indexer_logits_fp8 + torch.topk + ref_sparse_mla imported from oracle/_ref"
            if kind == "reference" else "the oracle's restatement of ref_indexer_logits_fp8 + torch.topk + ref_sparse_mla")
    sample = (f"{steps} full steps (ctx {args.ctx}, all {HEADS} heads, the whole layer on one host) after {warmup} warm-ups"
              f"{capped}; {what}; torch CPU, {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (e4m3/bf16 operands decoded on the host)",
        "data": "synthetic", "config": workload_config(args, max(world, args.gpus)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------ GPU arm
def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def event_time_ms(fn, iters):
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    st.record()
    for i in range(iters):
        fn(i)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


class LayerSet:
    """Per-layer caches and step buffers of one form of the hot path on this rank.

    form "replicated": every rank scans the whole key cache (the reference's scheme under TP,
    src/lagged_indexer_dsa/inference/modeling/transformer.py:673-677) and attends its own heads.
    form "sharded": rank r scans keys [r * ctx / N, (r + 1) * ctx / N); the ranks' local top-2048
    candidates are exchanged and merged (parallel.SeqShardedIndexer), then each rank attends its
    own heads over the merged selection."""

    def __init__(self, form, ctx, L, world, rank, dev, inputs, exchange="p2p"):
        from dsa_multi_layer_indexer_b200 import ops
        from dsa_multi_layer_indexer_b200.decode import HotPathState, LayerCache
        from dsa_multi_layer_indexer_b200.parallel import SeqShardedIndexer

        self.form, self.ctx, self.L, self.world, self.rank, self.dev = form, ctx, L, world, rank, dev
        self.sharded = form == "sharded" and world > 1
        self.heads_local = HEADS // world
        self.ctx_local = ctx // world if self.sharded else ctx
        key_lo = rank * self.ctx_local if self.sharded else 0
        h_iq8, h_w, h_q = inputs
        gen = torch.Generator(device=dev).manual_seed(1234)  # the same caches on every rank
        self.caches, self.states, self.indexers = [], [], []
        for _ in range(L):
            ik = torch.randn(ctx, 128, device=dev, generator=gen)
            ik8, sk = ops.quantize_e4m3_rowwise(ik)
            kv = torch.randn(ctx, 576, device=dev, generator=gen).to(torch.bfloat16)
            self.caches.append(LayerCache(ik8[key_lo:key_lo + self.ctx_local].unsqueeze(0).contiguous(),
                                          sk[key_lo:key_lo + self.ctx_local].unsqueeze(0).contiguous(), kv.unsqueeze(0)))
            del ik, ik8, sk
            st = HotPathState(1, self.heads_local, INDEX_HEADS, self.ctx_local, TOPK, dev)
            st.index_q.copy_(h_iq8)
            st.index_w.copy_(h_w)
            st.q.copy_(h_q[:, rank * self.heads_local:(rank + 1) * self.heads_local])
            if self.sharded:
                st.seq_lens.fill_(ctx)  # the attention sees the whole (replicated) latent cache
                self.indexers.append(SeqShardedIndexer(1, TOPK, self.ctx_local, key_lo, dev, exchange=exchange))
            self.states.append(st)
        torch.cuda.synchronize()

    def select(self, l, impl=0):
        st, cache = self.states[l], self.caches[l]
        if not self.sharded:
            return st.run_indexer(cache, impl)
        return self.indexers[l].select(st.index_q, st.index_w, cache.index_k, cache.k_scale)

    def step(self, l, impl=0):
        idx = self.select(l, impl)
        return self.states[l].run_attention(self.caches[l], idx, SM_SCALE)

    def free(self):
        for x in self.indexers:
            if x.xchg is not None:
                x.xchg.close()
        self.caches, self.states, self.indexers = [], [], []
        torch.cuda.empty_cache()


def time_steps(layers, steps, warmup, barrier, impl=0, graph_per_layer=False):
    """ms per step of `steps` consecutive layer steps, device-timed. A model's decode step is ONE
    graph over all its layers, so the timed loop replays a graph that holds L consecutive layer
    steps (L steps per replay, distinct caches); the steps beyond a multiple of L share one more."""
    L = layers.L
    for l in range(L):
        layers.step(l, impl)  # eager warm-up (opt-ins, lazy state)
    torch.cuda.synchronize()

    def capture(count):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(count):
                layers.step(l % L, impl)
        torch.cuda.synchronize()
        return g

    if graph_per_layer or L == 1:
        singles = [capture_one(layers, l, impl) for l in range(L)]
        plan = [(singles[i % L], 1) for i in range(steps)]
        warm = [singles[i % L] for i in range(max(warmup, 3))]
    else:
        n_big, rem = divmod(steps, L)
        big = capture(L) if n_big else None
        tail = capture(rem) if rem else None
        plan = [(big, L)] * n_big + ([(tail, rem)] if rem else [])
        warm = [g for g in (big, tail) if g is not None] * max(1, -(-max(warmup, 3) // L))
    barrier()
    for g in warm:
        g.replay()
    barrier()
    st_ev, en_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st_ev.record()
    for g, _ in plan:
        g.replay()
    en_ev.record()
    barrier()
    return st_ev.elapsed_time(en_ev) / steps


def capture_one(layers, l, impl=0):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        layers.step(l, impl)
    return g


def parity_check(world, rank, dev, ctx, inputs, dist):
    """Before anything is timed at N > 1: the N-rank result must be the one-GPU result on the same
    seeded inputs (the reference's own gate of this kind: batched == rows, bitwise,
    kernels/cuda_fused_sparse_splitk.py:3536-3668). Every rank runs both forms on one layer; rank 0
    also runs the whole layer alone and compares: selections exactly, the concatenated attention
    output within the 2e-2 bound (the split count of the attention depends on the head count, so
    its fp32 summation order differs). Returns (ok, max relative error of the attention)."""
    from dsa_multi_layer_indexer_b200 import _lib

    worst, ok = 0.0, True
    alone = None
    if rank == 0:
        ref = LayerSet("replicated", ctx, 1, 1, 0, dev, inputs)
        alone = (ref.select(0).clone(), ref.step(0).clone())
        ref.free()
    for form in ("replicated", "sharded"):
        ls = LayerSet(form, ctx, 1, world, rank, dev, inputs)
        sel = ls.select(0).clone()
        out = ls.states[0].run_attention(ls.caches[0], sel, SM_SCALE).clone()
        torch.cuda.synchronize()
        sels = [torch.empty_like(sel) for _ in range(world)]
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(sels, sel)
        dist.all_gather(outs, out)
        if rank == 0:
            ok = ok and all(torch.equal(s_, alone[0]) for s_ in sels)
            full = torch.cat(outs, dim=1).float()
            err = float((full - alone[1].float()).abs().max() / alone[1].float().abs().max())
            worst = max(worst, err)
            ok = ok and err < 2e-2
        ls.free()
        dist.barrier()
    _lib.check_device_status()
    flag = torch.tensor([1.0 if ok else 0.0, worst], dtype=torch.float64, device=dev)
    dist.broadcast(flag, 0)
    return bool(flag[0].item() > 0.5), float(flag[1].item())


def run_ours(args):
    import torch.distributed as dist

    from dsa_multi_layer_indexer_b200 import _lib, ops
    from dsa_multi_layer_indexer_b200.decode import HostDecoder

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()
    assert HEADS % world == 0
    ctx, L = args.ctx, args.layers

    # ---- the step's query operands come from (pinned) host memory
    hgen = torch.Generator().manual_seed(99)
    iq = torch.randn(1, INDEX_HEADS, 128, generator=hgen)
    w = torch.randn(1, INDEX_HEADS, generator=hgen) / 8
    q_all = torch.randn(1, HEADS, 576, generator=hgen).to(torch.bfloat16)
    iq8, sq = ops.quantize_e4m3_rowwise(iq.to(dev))
    h_iq8 = iq8.view(torch.uint8).cpu()
    h_w = (sq.cpu() * w).contiguous()
    inputs = (h_iq8.to(dev), h_w.to(dev), q_all.to(dev))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    parity = None
    if world > 1:
        ok, err = parity_check(world, rank, dev, ctx, inputs, dist)
        parity = {"parity_checked": ok, "parity_max_rel_err_attention": err,
                  "parity_note": "N-rank selection == one-GPU selection (exact) and concatenated attention output "
                                 "within 2e-2 of the one-GPU output, both forms, before the timed region"}
        if not ok:
            if rank == 0:
                print(json.dumps({"error": "the N-rank result differs from the one-GPU result", **parity}))
            dist.destroy_process_group()
            sys.exit(1)

    # the clock sampler starts early (nvidia-smi needs ~0.1 s to deliver its first sample)
    sampler = ClockSampler(local)
    sampler.start()

    forms = {}
    main = LayerSet("replicated", ctx, L, world, rank, dev, inputs)
    ms_rep = time_steps(main, args.steps, args.warmup, barrier, args.scan_impl, args.graph_per_layer)
    forms["tp_heads+replicated_indexer"] = ms_rep
    ms_shard = ms_shard2 = ms_rep2 = coll_ms = None
    if world > 1:
        sh = LayerSet("sharded", ctx, L, world, rank, dev, inputs)
        ms_shard = time_steps(sh, args.steps, args.warmup, barrier, args.scan_impl)
        # the exchange by itself: local top-k with the peer stores + the merge behind the bounded wait
        def xchg_only(l):
            x = sh.indexers[l]
            x.xchg.push(x.logits[:, :sh.ctx_local], None, hist=None, index_offset=x.key_lo)
            x.xchg.merge(x.indices)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(L):
                xchg_only(l)
        barrier()
        g.replay()
        barrier()
        reps = max(4, args.steps // L)
        st_ev, en_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st_ev.record()
        for _ in range(reps):
            g.replay()
        en_ev.record()
        barrier()
        coll_ms = st_ev.elapsed_time(en_ev) / (reps * L)
        del g
        sh.free()
        forms["tp_heads+seq_sharded_indexer"] = ms_shard
        if args.ctx == CTX:  # BASELINE config 5: the same step at twice the context
            sh2 = LayerSet("sharded", 2 * ctx, min(L, 8), world, rank, dev, inputs)
            ms_shard2 = time_steps(sh2, args.steps, args.warmup, barrier, args.scan_impl)
            sh2.free()
            forms["tp_heads+seq_sharded_indexer_ctx262144"] = ms_shard2
            rep2 = LayerSet("replicated", 2 * ctx, min(L, 8), world, rank, dev, inputs)  # the same length, every rank scanning all of it
            ms_rep2 = time_steps(rep2, args.steps, args.warmup, barrier, args.scan_impl)
            rep2.free()
            forms["tp_heads+replicated_indexer_ctx262144"] = ms_rep2
    ms_step = min(ms_rep, ms_shard) if ms_shard is not None else ms_rep
    best_form = "tp_heads+seq_sharded_indexer" if (ms_shard is not None and ms_shard < ms_rep) else \
        ("tp_heads+replicated_indexer" if world > 1 else "tp1_heads")

    # ---- each kernel alone, same rotation of caches: L launches back to back inside one graph, so the
    # figure is the kernel's own duration plus the in-graph launch gap, not the host's launch rate
    states, caches = main.states, main.caches

    def time_graphs(build):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(L):
                build(l)
        g.replay()
        reps = max(4, (max(args.steps, 64) + L - 1) // L)
        return event_time_ms(lambda i: g.replay(), reps) / L

    def scan_as_run(l):  # with its histogram epilogue, as the step runs it (each layer has its own histogram)
        s = states[l]
        ops.indexer_scan_fp8(s.index_q, s.index_w, caches[l].index_k, caches[l].k_scale, None,
                             ctx=ctx, out=s.logits, hist=s.hist, impl=args.scan_impl)

    def scan_nohist(l):
        s = states[l]
        ops.indexer_scan_fp8(s.index_q, s.index_w, caches[l].index_k, caches[l].k_scale, None,
                             ctx=ctx, out=s.logits, hist=None, impl=args.scan_impl)

    scan_ms = time_graphs(scan_as_run)
    for s in states:
        s.hist.zero_()  # (nothing re-armed them between those launches)
    scan_nohist_ms = time_graphs(scan_nohist)
    for s in states:  # a consistent histogram for the top-k leg below
        ops.indexer_scan_fp8(s.index_q, s.index_w, caches[0].index_k, caches[0].k_scale, None, ctx=ctx,
                             out=s.logits, hist=s.hist)
    torch.cuda.synchronize()

    def topk_as_run(l):  # consumes the scan's histogram and re-arms it: refill it by a copy node
        s = states[l]
        ops.topk_select(s.logits[:, :ctx], TOPK, None, hist=s.hist, out_idx=s.indices, workspace=s.topk_ws)
        s.hist.copy_(hist_keep[l])

    hist_keep = [s.hist.clone() for s in states]
    topk_copy_ms = time_graphs(topk_as_run)
    copy_ms = time_graphs(lambda l: states[l].hist.copy_(hist_keep[l]))
    topk_ms = topk_copy_ms - copy_ms
    for s in states:
        s.hist.zero_()
    attn_ms = time_graphs(lambda l: states[l].run_attention(caches[l], states[l].indices, SM_SCALE))

    def attn_stage(l, stage):
        s = states[l]
        ops.sparse_mla_decode(s.q, caches[l].kv, s.indices, SM_SCALE, s.seq_lens, scratch=s.scratch,
                              out=s.out, stage=stage)
    part_ms = time_graphs(lambda l: attn_stage(l, "partials"))
    comb_ms = time_graphs(lambda l: attn_stage(l, "combine"))
    # the lagged schedule's pair (attention over a given selection, this layer's indexer), as the
    # reference's own harness reports it (kernels/cuda_fused_sparse_splitk.py:4080-4094)
    attend = [s.indices.clone() for s in states]

    def indexer_only(l):
        states[l].run_indexer(caches[l], impl=args.scan_impl)

    def serial_pair(l):
        states[l].run_attention(caches[l], attend[l], SM_SCALE)
        states[l].run_indexer(caches[l], impl=args.scan_impl)

    def fused_pair(l):
        states[l].run_lagged_fused(caches[l], attend[l], SM_SCALE)

    side = torch.cuda.Stream(priority=-1)  # (high priority: 17.4 us against 19.5 us for the pair with a default-priority stream)

    def two_stream_pair(l):  # the default realisation: the indexer forks to a second stream and is joined
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            states[l].run_indexer(caches[l], impl=args.scan_impl)
        states[l].run_attention(caches[l], attend[l], SM_SCALE)
        cur.wait_stream(side)

    def chained_pair(l):  # one stream: scan, top-k, then the attention beside the top-k
        states[l].run_lagged_chained(caches[l], attend[l], SM_SCALE)

    idx_ms, ser_ms, fus_ms = time_graphs(indexer_only), time_graphs(serial_pair), time_graphs(fused_pair)
    two_ms = time_graphs(two_stream_pair)
    chain_ms = time_graphs(chained_pair)
    ideal = max(attn_ms, idx_ms)
    lag = {"attn_only_ms": attn_ms, "indexer_only_ms": idx_ms, "serial_ms": ser_ms, "fused_ms": fus_ms,
           "two_stream_ms": two_ms, "chained_ms": chain_ms, "ideal_overlap_ms": ideal,
           "fused_vs_ideal_pct": 100.0 * (fus_ms / ideal - 1.0),
           "two_stream_vs_ideal_pct": 100.0 * (two_ms / ideal - 1.0),
           "saved_vs_serial_pct": 100.0 * (1.0 - min(fus_ms, two_ms, chain_ms) / ser_ms),
           "note": "fused = one role-split launch (attention partials + indexer scan), then merge and top-k; "
                   "two_stream = indexer forked to a second, high-priority stream inside the graph (default realisation); "
                   "chained = one stream: scan, top-k, then the attention enqueued behind the top-k and running beside it; "
                   "with every kernel filling the device on its own, scan + max(top-k, attention) is the practical bound"}
    clocks = sampler.stop()

    # ---- end to end with host buffers (rank-local operands in pinned memory), over ALL the layer
    # caches, so that a step's keys are as cold as in the device-timed loop
    dec = [HostDecoder(states[l], caches[l], SM_SCALE) for l in range(L)]
    for d in dec:
        d.h_index_q.copy_(h_iq8)
        d.h_index_w.copy_(h_w)
        d.h_q.copy_(q_all[:, rank * main.heads_local:(rank + 1) * main.heads_local])
    for i in range(2 * L):
        dec[i % L].step()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        dec[i % L].step()
    barrier()
    e2e_dt = (time.perf_counter() - t0) / args.steps
    # The same steps with the next one enqueued before the host waits for the current one (each
    # decoder has its own pinned buffers): what a caller that is not itself in the data path between
    # steps gets. Reported beside the serial figure, which stays the headline.
    barrier()
    t0 = time.perf_counter()
    dec[0].launch()
    for i in range(1, args.steps):
        dec[i % L].launch()
        dec[(i - 1) % L].wait()
    dec[(args.steps - 1) % L].wait()
    barrier()
    e2e_pipe_dt = (time.perf_counter() - t0) / args.steps
    e2e = {"value": 1.0 / e2e_dt, "unit": UNIT, "ms_per_step": e2e_dt * 1e3,
           "h2d_bytes_per_step": dec[0].h2d_bytes, "d2h_bytes_per_step": dec[0].d2h_bytes,
           "form": "tp%d_heads%s" % (world, "+replicated_indexer" if world > 1 else ""),
           "pipelined_depth2_ms_per_step": e2e_pipe_dt * 1e3,
           "note": "one graph per step, cycling over all %d layer caches: index_q / index_w pinned host -> device by a "
                   "kernel node, q by the copy engine beside the scan, kernels, attention output written straight into pinned "
                   "host memory, selection -> pinned host by the graph's last node, which then posts the epoch word the "
                   "host polls, every step; pipelined_depth2 = the same steps with the next "
                   "step's graph enqueued before the host waits for the current one (this rank's wall clock)" % L}

    _lib.check_device_status()
    vals = [ms_step, scan_ms, topk_ms, attn_ms, e2e["ms_per_step"], ms_rep, ms_shard or 0.0, ms_shard2 or 0.0,
            coll_ms or 0.0, ms_rep2 or 0.0]
    times = torch.tensor(vals, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step, scan_ms, topk_ms, attn_ms, e2e_ms, ms_rep, ms_shard_m, ms_shard2_m, coll_m, ms_rep2_m = times.tolist()
    e2e["ms_per_step"] = e2e_ms
    e2e["value"] = 1e3 / e2e_ms
    if world > 1:
        ms_step = min(ms_rep, ms_shard_m)

    if rank == 0:
        peak, peak_src = measured_peaks()
        scan_bytes = ctx * SCAN_BYTES_PER_KEY
        achieved = scan_bytes / (scan_ms * 1e-3) / 1e9
        cfg = workload_config(args, world)
        out = {
            "metric": METRIC, "value": 1e3 / ms_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8 e4m3 (indexer MMA) + bf16 (MLA), fp32 accumulate",
            "data": "synthetic", "config": cfg, "form": best_form,
            "layer_us": ms_step * 1e3,
            "breakdown_us": {"indexer_scan": scan_ms * 1e3, "indexer_scan_without_histogram": scan_nohist_ms * 1e3,
                             "topk_select": topk_ms * 1e3,
                             "sparse_mla_partials_plus_combine": attn_ms * 1e3,
                             "sparse_mla_partials": part_ms * 1e3, "sparse_mla_combine": comb_ms * 1e3,
                             "note": "each kernel alone, as the step runs it (the scan with its histogram epilogue, the "
                                     "top-k consuming that histogram): L back-to-back launches (one per layer cache) inside "
                                     "one graph, includes the in-graph launch gap; measured on the replicated form"},
            "roofline": {"kernel": "indexer_scan_tc_kernel" if args.scan_impl == 0 else "indexer_scan_legacy_kernel",
                         "variant": "as the step runs it: with the histogram epilogue",
                         "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_src,
                         "frac_of_nominal_8TBs": achieved / 8000.0,
                         "frac_without_histogram": scan_bytes / (scan_nohist_ms * 1e-3) / 1e9 / peak,
                         "algorithmic_bytes_per_launch": scan_bytes,
                         "traffic": SCAN_TRAFFIC_CTX128K if (args.ctx == 131072 and args.scan_impl == 0) else None,
                         "traffic_source": "constant: dram__bytes_read.sum + dram__bytes_write.sum of one launch over "
                                           "131072 keys x 64 heads from an ncu capture (profiles/), not measured in this run"},
            "lagged_pair": lag,
            "gpu_launches": args.steps * (4 if best_form != "tp_heads+seq_sharded_indexer" else 5),
            "clocks": clocks,
            "e2e": e2e,
        }
        if world > 1:
            out["forms_ms_per_step"] = {k: v for k, v in
                                        (("tp_heads+replicated_indexer", ms_rep), ("tp_heads+seq_sharded_indexer", ms_shard_m),
                                         ("tp_heads+seq_sharded_indexer_ctx262144", ms_shard2_m),
                                         ("tp_heads+replicated_indexer_ctx262144", ms_rep2_m)) if v}
            out["collective_us"] = coll_m * 1e3
            out["comm"] = ("sharded form: every step stores this rank's 2048 (index, logit) candidates into all ranks' gather "
                           "buffers over NVLink (peer stores, no NCCL call, no multicast) and waits on the device for the "
                           "others' flags: inside the timed region, inside the graph; collective_us = local top-k + stores + "
                           "wait + merge per step. Replicated form: no collective (the selection is deterministic)")
            out.update(parity)
        if not args.no_cpu_baseline and world == 1:
            dt, cores, kind = time_cpu(ctx, 10, 2)
            out["cpu_baseline"] = {"value": 1.0 / dt, "unit": UNIT, "cores": cores, "kind": kind,
                                   "sample": f"10 full steps (ctx {ctx}, 128 heads) after 2 warm-ups, torch CPU"}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------ other BASELINE configs
# (parity-test cases, measured on request; the default line above stays config 2)
def _timed_graph(fn, reps):
    """Captures fn() once, replays reps times, returns ms per replay (CUDA events)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    return event_time_ms(lambda i: g.replay(), reps)


def run_batch32_paged(args):
    """BASELINE config 4: batch 32, lengths ~U[16384, 65536], page-64 index keys,
    fp8-packed latent rows, ragged split-K."""
    from dsa_multi_layer_indexer_b200 import _lib, ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, cap = 32, 65536
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16384, 65537, (B,), generator=g, dtype=torch.int32)
    pages_per = cap // 64
    num_pages = B * pages_per
    perm = torch.randperm(num_pages, generator=g).int().view(B, pages_per)
    gen = torch.Generator(device=dev).manual_seed(1)
    pool = torch.empty(num_pages, 8448, dtype=torch.uint8, device=dev)
    kv_rows = torch.empty(B, cap, 656, dtype=torch.uint8, device=dev)
    for b in range(B):  # quantise on the device, then scatter into pages / packed rows
        ik8, sk = ops.quantize_e4m3_rowwise(torch.randn(cap, 128, device=dev, generator=gen))
        pg = pool[perm[b].long().to(dev)]
        pg[:, :8192] = ik8.view(torch.uint8).view(pages_per, 8192)
        pg[:, 8192:] = sk.view(pages_per, 64).contiguous().view(torch.uint8).view(pages_per, 256)
        pool[perm[b].long().to(dev)] = pg
        lat = torch.randn(cap, 576, device=dev, generator=gen)
        q8, s8 = ops.quantize_e4m3_rowwise(lat[:, :512].reshape(cap * 4, 128).contiguous(), clamp_min=1e-4)
        kv_rows[b, :, :512] = q8.view(torch.uint8).view(cap, 512)
        kv_rows[b, :, 512:528] = s8.view(cap, 4).contiguous().view(torch.uint8).view(cap, 16)
        kv_rows[b, :, 528:] = lat[:, 512:].to(torch.bfloat16).contiguous().view(torch.uint8).view(cap, 128)
    iq8, sq = ops.quantize_e4m3_rowwise(torch.randn(B, INDEX_HEADS, 128, device=dev, generator=gen))
    w = (sq * torch.randn(B, INDEX_HEADS, device=dev, generator=gen) / 8).contiguous()
    q = torch.randn(B, HEADS, 576, device=dev, generator=gen).to(torch.bfloat16)
    seq = lens.to(dev)
    pt = perm.to(dev)
    logits = torch.empty(B, cap, dtype=torch.float32, device=dev)
    hist = torch.zeros(B, ops.HIST_BINS, dtype=torch.int32, device=dev)
    ws = ops.topk_workspace(B, cap, dev)
    idx = torch.empty(B, TOPK, dtype=torch.int32, device=dev)
    nsplit = ops.default_nsplit(B, HEADS, TOPK)
    scratch = ops.MlaScratch(B, HEADS, nsplit, dev)
    out = torch.empty(B, HEADS, 512, dtype=torch.bfloat16, device=dev)

    def scan():
        return ops.indexer_scan_fp8_paged(iq8, w, pool, pt, seq, cap, out=logits, hist=hist)

    def select():
        ops.topk_select(logits, TOPK, seq, hist=hist, out_idx=idx, workspace=ws)

    def attend():
        ops.sparse_mla_decode(q, kv_rows, idx, SM_SCALE, seq, scratch=scratch, out=out)

    def step():
        scan()
        select()
        attend()

    step()
    torch.cuda.synchronize()
    reps = max(8, args.steps // 8)
    ms = _timed_graph(step, reps)
    scan_ms = _timed_graph(lambda: (scan(), hist.zero_()), reps)  # (the top-k re-arms the histogram in a real step)
    scan_plain_ms = _timed_graph(lambda: ops.indexer_scan_fp8_paged(iq8, w, pool, pt, seq, cap, out=logits), reps)
    sel_ms = _timed_graph(lambda: (scan(), select()), reps) - scan_plain_ms
    att_ms = _timed_graph(attend, reps)
    _lib.check_device_status()
    peak, src = measured_peaks()
    scan_bytes = int(lens.sum()) * SCAN_BYTES_PER_KEY
    ach = scan_bytes / (scan_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "dsa_decode_layer_tokens_per_s_batch32_paged", "value": B * 1e3 / ms, "unit": UNIT, "n_gpus": 1,
        "steps": reps, "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8 e4m3 indexer + fp8-packed latent rows dequantised to bf16", "data": "synthetic",
        "config": {"workload": "batch32_ragged_paged_fp8_latent (BASELINE config 4)", "batch": B,
                   "lens": "U[16384,65536] seed 0, sum %d" % int(lens.sum()), "page_tokens": 64, "topk": TOPK,
                   "mla_heads": HEADS, "nsplit": nsplit,
                   "l2": "one step reads %.0f MB of index pages: larger than L2" % (scan_bytes / 1e6)},
        "breakdown_us": {"indexer_scan_paged_with_hist_plus_memset": scan_ms * 1e3,
                         "indexer_scan_paged_without_histogram": scan_plain_ms * 1e3,
                         "topk_select_plus_the_scans_histogram_epilogue": sel_ms * 1e3,
                         "sparse_mla_fp8_rows": att_ms * 1e3},
        "roofline": {"kernel": "indexer_scan_tc_kernel (paged)", "bound": "hbm", "achieved": ach, "peak": peak,
                     "unit": "GB/s", "frac": ach / peak, "peak_source": src,
                     "algorithmic_bytes_per_launch": scan_bytes, "traffic": None},
        "gpu_launches": reps * 5,
    }))


def run_mli_stack(args):
    """BASELINE config 3: 8 DSA layers (hidden 7168, 128 heads, MLP 18432, bf16), batch 1, context 131072, FP8 index
    keys: BASELINE order vs the lagged schedule with the indexer on a second stream, each step one CUDA graph.
    Under torchrun the stack is tensor-parallel over the ranks (heads and MLP columns split, the partial outputs of
    o_proj / down_proj all-reduced by peer stores inside the graph, indexer replicated)."""
    import torch.distributed as dist

    import dsa_multi_layer_indexer_b200 as D
    from dsa_multi_layer_indexer_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_layers, ctx = 8, args.ctx
    cfg = D.DSAConfig(num_hidden_layers=n_layers, first_k_dense_replace=0)
    torch.manual_seed(rank)
    if world > 1:
        model = D.DSAModel.tensor_parallel(cfg, None, dev, dtype=torch.bfloat16)
    else:
        with torch.device(dev):
            model = D.DSAModel(cfg).to(torch.bfloat16).eval()
    gen = torch.Generator(device=dev).manual_seed(2)  # the same caches and token on every rank

    def fresh_state(retention=None):
        st = model.init_decode(1, ctx, fp8=True, retention=retention)
        for c in st.caches:  # synthetic prefix of ctx - 1 tokens instead of a 128K-token prefill
            c.index_k.copy_(torch.randint(0, 120, c.index_k.shape, device=dev, generator=gen, dtype=torch.uint8))
            c.k_scale.copy_(torch.rand(c.k_scale.shape, device=dev, generator=gen) * 0.01 + 0.005)
            c.kv.copy_(torch.randn(c.kv.shape, device=dev, generator=gen).to(torch.bfloat16))
        st.positions.fill_(ctx - 1)
        st.seq_lens.fill_(ctx - 1)
        return st

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results = {}
    reps = max(8, args.steps // 16)
    x = torch.randn(1, cfg.hidden_size, device=dev, generator=gen).to(torch.bfloat16)
    for name, mode, overlap, retention in (
            ("baseline_serial", D.ScheduleMode.BASELINE, False, None),
            ("lagged_one_stream", D.ScheduleMode.LAGGED_FUSED, False, None),
            ("lagged_two_streams", D.ScheduleMode.LAGGED_FUSED, True, None),
            ("lagged_chained_one_stream", D.ScheduleMode.LAGGED_FUSED, "chained", None),
            ("lagged_two_streams_retention_1of4", D.ScheduleMode.LAGGED_FUSED, True, "4"),
            ("lagged_one_indexer_in_8_layers", D.ScheduleMode.LAGGED_FUSED, False, "8")):
        st = fresh_state(retention)
        graph, x_in, _ = model.capture_decode(st, mode, D.ColdStartPolicy.EAGER, overlap=overlap)
        x_in.copy_(x)
        saved = (st.positions.clone(), st.seq_lens.clone())

        def replay(i):
            graph.replay()
            st.positions.copy_(saved[0])  # stay at the same context length
            st.seq_lens.copy_(saved[1])

        for i in range(3):
            replay(i)
        barrier()
        results[name] = event_time_ms(replay, reps) * 1e3 / n_layers
        barrier()
        if name == "lagged_one_stream":  # the indexer branch alone: every layer's scan + top-k on the operands
            lay_ops = []               # the step above left in place, back to back in one graph
            for li, layer in enumerate(model.layers):
                ws = st.workspaces[li]
                iq = torch.randint(0, 120, (1, cfg.index_n_heads, cfg.index_head_dim), device=dev, generator=gen,
                                   dtype=torch.uint8)
                wv = torch.rand(1, cfg.index_n_heads, device=dev, generator=gen) * 0.01
                lay_ops.append((layer, iq, wv, st.caches[li], ws))
            g2 = torch.cuda.CUDAGraph()
            for layer, iq, wv, cache, ws in lay_ops:
                layer.decode_indexer(iq, wv, cache, st.seq_lens, ws=ws)
            torch.cuda.synchronize()
            with torch.cuda.graph(g2):
                for layer, iq, wv, cache, ws in lay_ops:
                    layer.decode_indexer(iq, wv, cache, st.seq_lens, ws=ws)
            g2.replay()
            results["indexer_branch"] = event_time_ms(lambda i: g2.replay(), reps) * 1e3 / n_layers
            del g2, lay_ops
        del graph, st
        torch.cuda.empty_cache()
    _lib.check_device_status()
    vals = torch.tensor([results[k] for k in sorted(results)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    results = dict(zip(sorted(results), vals.tolist()))
    lag = min(results["lagged_two_streams"], results["lagged_chained_one_stream"])
    idx_us = results["indexer_branch"]
    # attention + MLP of a layer: the stack with ONE indexer in its 8 layers, minus that indexer's share
    attn_mlp_us = results["lagged_one_indexer_in_8_layers"] - idx_us / n_layers
    max_us = max(idx_us, attn_mlp_us)
    if rank == 0:
        print(json.dumps({
            "metric": "dsa_mli_layer_latency_us_ctx128k", "value": lag, "unit": "us/layer", "n_gpus": world, "steps": reps,
            "warmup": 3, "ms_per_step": lag * n_layers / 1e3, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 weights/activations, fp8 e4m3 index keys", "data": "synthetic",
            "config": {"workload": "mli_lagged_8_layer_stack (BASELINE config 3)",
                       "parallelism": "tp%d: MLA heads and MLP columns split, o_proj / down_proj partial sums all-reduced by "
                                      "peer stores inside the graph, indexer replicated" % world if world > 1 else "tp1",
                       "layers": n_layers, "context": ctx,
                       "hidden": cfg.hidden_size, "mla_heads_per_gpu": cfg.num_attention_heads // world,
                       "intermediate_per_gpu": cfg.intermediate_size // world,
                       "weights_GB_per_layer_per_gpu": sum(p.numel() for p in model.layers[0].parameters()) * 2 / 1e9,
                       "l2": "the layer's weights + 168 MB of caches per layer: larger than L2"},
            "us_per_layer": results,
            "indexer_branch_us": idx_us, "attention_plus_mlp_us": attn_mlp_us, "max_us": max_us,
            "overlapped_us": lag, "overlapped_vs_max_pct": 100.0 * (lag / max_us - 1.0),
            "serial_us": results["baseline_serial"],
            "overlapped_form": ("chained_one_stream" if results["lagged_chained_one_stream"] <= results["lagged_two_streams"]
                                else "two_streams"),
            "note": "one CUDA graph per decode step; overlapped = the faster of the two lagged realisations (indexer on a "
                    "second stream; or one stream with the attention enqueued behind the layer's scan and top-k and running "
                    "beside the top-k); per-layer figure = step / 8; projections and MLP are cuBLAS/torch; "
                    "indexer_branch = scan + top-k of every layer back to back in one graph / 8; attention_plus_mlp = the "
                    "lagged stack with one indexer in its 8 layers minus that indexer's share; target: overlapped within "
                    "10 % of max(indexer_branch, attention_plus_mlp)",
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "batch32_paged":
        run_batch32_paged(args)
    elif args.workload == "mli_stack":
        run_mli_stack(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
