"""Serving-form indexer staging (``dsa_indexer_stage_fp8``) against the oracle and
the reference-made fixtures: LayerNorm of the key, rotary embedding, Hadamard
rotation, act_quant, folded head weights and the cache append
(inference/modeling/transformer.py:1015-1066 in the reference)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_golden
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def D():
    from dsa_multi_layer_indexer_b200 import ops
    return ops


def _inputs(B, H, cap, seed):
    g = torch.Generator().manual_seed(seed)
    q_raw = torch.randn(B, H, 128, generator=g).to(torch.bfloat16)
    k_raw = (torch.randn(B, 128, generator=g) * 2 + 0.3).to(torch.bfloat16)
    w_raw = torch.randn(B, H, generator=g)
    ang = torch.rand(cap, 32, generator=g) * 6.2831853
    norm_w = 1 + 0.1 * torch.randn(128, generator=g)
    norm_b = 0.05 * torch.randn(128, generator=g)
    positions = torch.randint(0, cap, (B,), generator=g)
    return q_raw, k_raw, w_raw, torch.cos(ang), torch.sin(ang), norm_w, norm_b, positions


def _run_dense(D, q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions, inter, fmt, cap):
    dev = "cuda"
    B, H, _ = q_raw.shape
    index_q = torch.zeros(B, H, 128, dtype=torch.uint8, device=dev)
    index_w = torch.zeros(B, H, device=dev)
    cache_k = torch.full((B, cap, 128), 0x55, dtype=torch.uint8, device=dev)
    cache_s = torch.full((B, cap), -1.0, device=dev)
    D.indexer_stage_fp8(q_raw.to(dev), k_raw.to(dev), w_raw.to(dev), norm_w.to(dev), norm_b.to(dev), 1e-6,
                        cos.to(dev), sin.to(dev), positions.to(dev), index_q, index_w, cache_k, cache_s,
                        rope_interleave=inter, scale_fmt=fmt)
    torch.cuda.synchronize()
    return index_q.cpu(), index_w.cpu(), cache_k.cpu(), cache_s.cpu()


@pytest.mark.parametrize("inter", [False, True])
@pytest.mark.parametrize("fmt", [None, "ue8m0"])
@pytest.mark.parametrize("B,H", [(1, 64), (5, 64), (3, 32)])
def test_stage_matches_oracle(D, inter, fmt, B, H):
    cap = 512
    q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions = _inputs(B, H, cap, seed=B * 100 + H)
    index_q, index_w, cache_k, cache_s = _run_dense(D, q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions,
                                                    inter, fmt, cap)
    q8, w, k8, ks = O.indexer_stage_fp8(q_raw, k_raw, w_raw, norm_w, norm_b, 1e-6, cos, sin, positions.tolist(),
                                        inter, fmt is not None, 128 ** -0.5)
    # query path: the same rounded operations in the same order -> the same bytes and weights
    assert torch.equal(index_q, q8)
    assert torch.equal(index_w, w)
    # key path: LayerNorm's fp32 summation order differs from torch's, so a bf16 may
    # round the other way now and then; dequantised keys agree to within one e4m3 step.
    rows = torch.arange(B)
    got_k, got_s = cache_k[rows, positions], cache_s[rows, positions]
    assert torch.allclose(got_s, ks, rtol=2 ** -7, atol=0)
    deq_g = O.e4m3_to_f32(got_k) * got_s.unsqueeze(-1)
    deq_o = O.e4m3_to_f32(k8) * ks.unsqueeze(-1)
    step = deq_o.abs() * 2 ** -3 + ks.unsqueeze(-1) * 2 ** -9
    assert ((deq_g - deq_o).abs() <= step * 1.01).all()
    assert (got_k == k8).float().mean() > 0.97
    # nothing else in the cache was touched
    untouched = torch.ones(B, cap, dtype=torch.bool)
    untouched[rows, positions] = False
    assert cache_k[untouched].eq(0x55).all() and cache_s[untouched].eq(-1.0).all()


def test_stage_against_reference_fixture(D):
    """Dequantised GPU operands against the rotated bf16 operands the reference's own
    LayerNorm / apply_rotary_emb / rotate_activation produced."""
    g = load_golden("indexer_stage.npz")
    q_raw, k_raw = bf16_from_bits(g["q_raw"]), bf16_from_bits(g["k_raw"])
    B, H, _ = q_raw.shape
    cos, sin = torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"])
    norm_w, norm_b = torch.from_numpy(g["norm_w"]), torch.from_numpy(g["norm_b"])
    w_raw = torch.ones(B, H)
    positions = torch.arange(B)
    for inter in (False, True):
        index_q, index_w, cache_k, cache_s = _run_dense(D, q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b,
                                                        positions, inter, None, B)
        q_scale = index_w / (H ** -0.5 * 128 ** -0.5)
        q_rot = bf16_from_bits(g[f"q_rot_{int(inter)}"]).float()
        k_rot = bf16_from_bits(g[f"k_rot_{int(inter)}"]).float()
        deq_q = O.e4m3_to_f32(index_q) * q_scale.unsqueeze(-1)
        assert ((deq_q - q_rot).abs() <= q_rot.abs() * 2 ** -4 + q_scale.unsqueeze(-1) * 2 ** -10 * 1.01).all()
        ks = cache_s[positions, positions]
        deq_k = O.e4m3_to_f32(cache_k[positions, positions]) * ks.unsqueeze(-1)
        # one bf16 step of slack on top of the quantisation step (LayerNorm summation order)
        assert ((deq_k - k_rot).abs() <= k_rot.abs() * (2 ** -4 + 2 ** -7) + ks.unsqueeze(-1) * 2 ** -9).all()


def test_stage_paged_append_equals_dense(D):
    dev = "cuda"
    B, H, cap = 4, 64, 256
    q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions = _inputs(B, H, cap, seed=9)
    _, _, cache_k, cache_s = _run_dense(D, q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions, False, None, cap)
    pages_per_seq = cap // 64
    n_pages = B * pages_per_seq + 3
    perm = torch.randperm(n_pages)[: B * pages_per_seq].to(torch.int32).view(B, pages_per_seq)
    pages = torch.full((n_pages * 8448,), 0x55, dtype=torch.uint8, device=dev)
    index_q = torch.zeros(B, H, 128, dtype=torch.uint8, device=dev)
    index_w = torch.zeros(B, H, device=dev)
    D.indexer_stage_fp8(q_raw.to(dev), k_raw.to(dev), w_raw.to(dev), norm_w.to(dev), norm_b.to(dev), 1e-6,
                        cos.to(dev), sin.to(dev), positions.to(dev), index_q, index_w, pages=pages,
                        page_table=perm.to(dev))
    torch.cuda.synchronize()
    pg = pages.cpu().view(n_pages, 8448)
    touched = 0
    for b in range(B):
        pos = int(positions[b])
        page = pg[int(perm[b, pos // 64])]
        assert torch.equal(page[(pos % 64) * 128:(pos % 64 + 1) * 128], cache_k[b, pos])
        assert page[64 * 128 + (pos % 64) * 4: 64 * 128 + (pos % 64) * 4 + 4].view(torch.float32)[0] == cache_s[b, pos]
        touched += 132
    assert int((pg != 0x55).sum()) <= touched


def test_staged_operands_feed_the_scan(D):
    """Staging a run of tokens one by one, then scanning: logits equal the oracle's
    on its own staged operands (same bytes in, so only the fp32 summation order differs)."""
    dev = "cuda"
    H, cap, T = 64, 256, 200
    g = torch.Generator().manual_seed(21)
    ang = torch.rand(cap, 32, generator=g) * 6.2831853
    cos, sin = torch.cos(ang), torch.sin(ang)
    norm_w, norm_b = 1 + 0.1 * torch.randn(128, generator=g), 0.05 * torch.randn(128, generator=g)
    cache_k = torch.zeros(1, cap, 128, dtype=torch.uint8, device=dev)
    cache_s = torch.zeros(1, cap, device=dev)
    index_q = torch.zeros(1, H, 128, dtype=torch.uint8, device=dev)
    index_w = torch.zeros(1, H, device=dev)
    for t in range(T):
        q_raw = torch.randn(1, H, 128, generator=g).to(torch.bfloat16)
        k_raw = torch.randn(1, 128, generator=g).to(torch.bfloat16)
        w_raw = torch.randn(1, H, generator=g)
        D.indexer_stage_fp8(q_raw.to(dev), k_raw.to(dev), w_raw.to(dev), norm_w.to(dev), norm_b.to(dev), 1e-6,
                            cos.to(dev), sin.to(dev), torch.tensor([t], device=dev), index_q, index_w, cache_k, cache_s)
    torch.cuda.synchronize()
    seq_lens = torch.tensor([T], dtype=torch.int32, device=dev)
    logits = D.indexer_scan_fp8(index_q, index_w, cache_k, cache_s, seq_lens)
    torch.cuda.synchronize()
    ref = O.indexer_logits_fp8(index_q.cpu(), cache_k.cpu()[0, :T], index_w.cpu(), cache_s.cpu()[0, :T])[0]
    got = logits.cpu()[0, :T]
    assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()
    assert torch.isinf(logits.cpu()[0, T:]).all()
