"""In-situ timeline of the hot path from the tracing build of the library.

    python -m dsa_multi_layer_indexer_b200.trace [--ctx 131072] [--heads 128] [--layers 4]

Builds the library with ``-DDSA_STAMPS`` next to the normal one, loads it
instead (the same C ABI), replays one captured step per layer cache and prints,
per kernel, begin and end in microseconds from the first scan CTA's start (the
kernels stamp ``%globaltimer``; read back with ``dsa_debug_read_stamps``). The
reference has the same facility behind ``hide_debug_enable`` / ``hide_debug_read``
(kernels/cuda_fused_sparse_splitk.py:1076-1090, :2329-2349).
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

KERNELS = {0: "indexer_scan", 1: "topk_cluster", 2: "sparse_mla_partials", 3: "sparse_mla_combine"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--reps", type=int, default=6)
    args = ap.parse_args()

    from .csrc import build as _build

    trace_lib = Path(_build.PKG) / "libdsa_b200_trace.so"
    _build.build_trace(trace_lib)
    os.environ["DSA_B200_LIB"] = str(trace_lib)

    import numpy as np
    import torch

    from . import _lib, ops
    from .decode import HotPathState, LayerCache

    if _lib._lib is not None:
        raise RuntimeError("the library is already loaded; run the tracer in a fresh process")
    _lib.LIB_PATH = trace_lib  # same ABI, with stamps
    lib = _lib.lib()
    dev = "cuda"
    n_words = 1024 * 16 + 32

    def read():
        buf = np.zeros(n_words, dtype=np.uint64)
        rc = lib.dsa_debug_read_stamps(buf.ctypes.data, buf.size)
        if rc < 0:
            _lib.check(rc)
        return buf[1024 * 16:].astype(np.int64)

    torch.manual_seed(0)
    caches, states, graphs = [], [], []
    for _ in range(args.layers):
        ik8, sk = ops.quantize_e4m3_rowwise(torch.randn(args.ctx, 128, device=dev))
        kv = torch.randn(args.ctx, 576, device=dev).to(torch.bfloat16)
        caches.append(LayerCache(ik8.unsqueeze(0).contiguous(), sk.unsqueeze(0).contiguous(), kv.unsqueeze(0)))
        st = HotPathState(1, args.heads, 64, args.ctx, 2048, dev)
        iq8, sq = ops.quantize_e4m3_rowwise(torch.randn(1, 64, 128, device=dev))
        st.index_q.copy_(iq8.view(torch.uint8))
        st.index_w.copy_(sq * torch.randn(1, 64, device=dev) / 8)
        st.q.copy_(torch.randn(1, args.heads, 576, device=dev).to(torch.bfloat16))
        states.append(st)
    for st, cache in zip(states, caches):
        graphs.append(st.capture(cache, 192 ** -0.5))
    torch.cuda.synchronize()
    for rep in range(args.reps):
        for l, g in enumerate(graphs):
            read()
            g.replay()
            torch.cuda.synchronize()
            t = read()
            if rep == args.reps - 1:
                t0 = t[0]
                row = "  ".join(f"{name} [{(t[2 * k] - t0) / 1e3:5.2f}, {(t[2 * k + 1] - t0) / 1e3:5.2f}]"
                                for k, name in KERNELS.items())
                print(f"layer cache {l}: {row}  (us)")
    _lib.check_device_status()


if __name__ == "__main__":
    sys.exit(main())
