"""The reference extension's launch functions (same names, same argument lists)
bound to libdsa_b200.so, exercised the way the reference's own validate() and
validate_batched() exercise them (kernels/cuda_fused_sparse_splitk.py:3072-3105,
:3536-3668), with the tolerances tightened to this build's targets."""

from __future__ import annotations

import pytest
import torch

from conftest import corr_diff, rel_err
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


def make_case(S, Skv, H, Hidx, topk, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, H, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(1, Skv, 1, 576, generator=g).to(torch.bfloat16)
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(torch.randn(S, Hidx, 128, generator=g),
                                                 torch.randn(Skv, 128, generator=g),
                                                 torch.randn(S, Hidx, generator=g).abs())
    idx = torch.full((S, topk), Skv, dtype=torch.int32)
    for s in range(S):
        prefix = (Skv - S) + s + 1
        take = min(topk, prefix)
        idx[s, :take] = torch.randperm(prefix, generator=g)[:take].int()
    return q, kv, idx, iq8, ik8, wp, sk


@pytest.mark.parametrize("S,Skv,H,nsplit", [(1, 4096, 16, 8), (4, 5000, 32, 4), (2, 2048, 128, 32)])
def test_launch_fused_sparse_splitk_like_validate(S, Skv, H, nsplit):
    from dsa_multi_layer_indexer_b200 import kernels_ext as K

    ext = K.build()
    topk, Hidx = 2048, 64
    q, kv, idx, iq8, ik8, wp, sk = make_case(S, Skv, H, Hidx, topk, seed=S + H)
    dev = "cuda"
    out = torch.zeros(1, S, H, 512, dtype=torch.bfloat16, device=dev)
    slab = torch.zeros(S, Skv, dtype=torch.float32, device=dev)
    hist = torch.zeros(S, 4096, dtype=torch.int32, device=dev)
    pa, pm, pl = K.alloc_part(S, H, nsplit, dev)
    sm = 576 ** -0.5
    ext.launch_fused_sparse_splitk(q.to(dev), kv.to(dev), idx.to(dev), iq8.to(dev), ik8.to(dev), wp.to(dev),
                                   sk.to(dev), pa, pm, pl, slab, hist, out, S, Skv, H, Hidx, topk, nsplit, sm, 2, 1, 0)
    torch.cuda.synchronize()
    lens = [(Skv - S) + s + 1 for s in range(S)]
    ref_out = O.sparse_mla_decode(q[0], kv[0, :, 0], idx, lens, sm)
    assert corr_diff(out[0].float().cpu(), ref_out) < 1e-3
    assert rel_err(out[0].float().cpu(), ref_out) < 2e-2
    ref_logits = O.mask_beyond(O.indexer_logits_fp8(iq8, ik8, wp, sk), lens)
    fin = torch.isfinite(ref_logits)
    got = slab.cpu()
    assert torch.equal(torch.isfinite(got), fin)
    assert rel_err(got[fin], ref_logits[fin]) < 1e-2
    assert hist.sum(1).cpu().tolist() == lens  # with_select=2: the histogram counts every causal key


def test_batched_launch_equals_single_row_launches_bitwise():
    from dsa_multi_layer_indexer_b200 import kernels_ext as K

    ext = K.build()
    B, Skv, H, Hidx, topk, nsplit = 3, 3000, 32, 64, 1024, 8
    dev = "cuda"
    torch.manual_seed(3)
    q = torch.randn(1, B, H, 576).to(torch.bfloat16).to(dev)
    kv = torch.randn(B, Skv, 576).to(torch.bfloat16).to(dev)
    idx = torch.stack([torch.randperm(Skv)[:topk] for _ in range(B)]).int().to(dev)
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, Hidx, 128))
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, Skv, 128))
    wp = (sq * torch.randn(B, Hidx).abs()).to(dev)
    iq8, ik8, sk = iq8.to(dev), ik8.to(dev), sk.to(dev)
    sm = 576 ** -0.5

    def launch(rows):
        n = len(rows)
        out = torch.zeros(1, n, H, 512, dtype=torch.bfloat16, device=dev)
        slab = torch.zeros(n, Skv, dtype=torch.float32, device=dev)
        pa, pm, pl = K.alloc_part(n, H, nsplit, dev)
        r = torch.tensor(rows, device=dev)
        ext.launch_fused_sparse_splitk_batch_idx(
            q[:, r].contiguous(), kv[r].contiguous(), idx[r].contiguous(), iq8[r].contiguous(), ik8[r].contiguous(),
            wp[r].contiguous(), sk[r].contiguous(), pa, pm, pl, slab, None, out, n, Skv, H, Hidx, topk, nsplit, sm,
            1, 1, 0, Skv * 576, Skv * 128, Skv)
        torch.cuda.synchronize()
        return out[0], slab

    out_all, slab_all = launch([0, 1, 2])
    for b in range(B):
        o, s = launch([b])
        assert torch.equal(o[0], out_all[b])
        assert torch.equal(s[0], slab_all[b])
    with pytest.raises(RuntimeError):
        ext.launch_fused_sparse_splitk(None, None, None, None, None, None, None, None, None, None, None, None, None,
                                       1, 1, 16, 64, 2048, 1, 1.0, 4, 1, 0)
