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


def test_stage_and_scan_do_not_follow_a_bad_page_table_entry(D):
    """A page-table entry of -1 (or one beyond the pool) must not become a wild access: the
    staging kernel skips that token and leaves every pool byte as it was, the paged scan gives
    the keys behind such an entry logit -inf, and both report through the device status word."""
    from dsa_multi_layer_indexer_b200 import _lib

    dev = "cuda"
    B, H, cap = 3, 64, 256
    q_raw, k_raw, w_raw, cos, sin, norm_w, norm_b, positions = _inputs(B, H, cap, seed=21)
    pages_per_seq = cap // 64
    n_pages = B * pages_per_seq
    perm = torch.randperm(n_pages).to(torch.int32).view(B, pages_per_seq)
    bad = perm.clone()
    bad[1, int(positions[1]) // 64] = -1          # the page sequence 1 would append to
    bad[2, int(positions[2]) // 64] = n_pages + 5  # beyond the pool
    pages = torch.full((n_pages * 8448,), 0x55, dtype=torch.uint8, device=dev)
    index_q = torch.zeros(B, H, 128, dtype=torch.uint8, device=dev)
    index_w = torch.zeros(B, H, device=dev)
    _lib.check_device_status()
    D.indexer_stage_fp8(q_raw.to(dev), k_raw.to(dev), w_raw.to(dev), norm_w.to(dev), norm_b.to(dev), 1e-6,
                        cos.to(dev), sin.to(dev), positions.to(dev), index_q, index_w, pages=pages,
                        page_table=bad.to(dev))
    with pytest.raises(_lib.DsaError) as err:
        _lib.check_device_status()
    assert err.value.status == -1 and "page-table" in str(err.value)
    _lib.check_device_status()  # the word was cleared by the read
    pg = pages.cpu().view(n_pages, 8448)
    assert int((pg != 0x55).sum()) <= 132  # only sequence 0's token was written
    pos0 = int(positions[0])
    assert bool((pg[int(perm[0, pos0 // 64])][(pos0 % 64) * 128:(pos0 % 64 + 1) * 128] != 0x55).any())
    # the paged scan: keys behind a bad entry get -inf, every other logit is what the good table gives
    g = torch.Generator().manual_seed(5)
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, cap, 128, generator=g))
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, H, 128, generator=g))
    wp = sq * (torch.randn(B, H, generator=g) / 8)
    pool = torch.zeros(n_pages, 8448, dtype=torch.uint8)
    for b in range(B):
        O.pack_index_pages(ik8[b], sk[b], perm[b].tolist(), n_pages, pool)
    lens = torch.full((B,), cap, dtype=torch.int32, device=dev)
    good = D.indexer_scan_fp8_paged(iq8.to(dev), wp.to(dev), pool.to(dev), perm.to(dev), lens, cap).cpu()
    _lib.check_device_status()
    got = D.indexer_scan_fp8_paged(iq8.to(dev), wp.to(dev), pool.to(dev), bad.to(dev), lens, cap).cpu()
    with pytest.raises(_lib.DsaError):
        _lib.check_device_status()
    for b in range(B):
        for pidx in range(pages_per_seq):
            span = slice(pidx * 64, pidx * 64 + 64)
            if int(bad[b, pidx]) != int(perm[b, pidx]):
                assert torch.isinf(got[b, span]).all() and (got[b, span] < 0).all()
            else:
                assert torch.equal(got[b, span], good[b, span])


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


# ------------------------------------------------------------------ latent append
def _latent_inputs(B, cap, n_slots, seed):
    g = torch.Generator().manual_seed(seed)
    kv_a = (torch.randn(B, 576, generator=g) * 1.5).to(torch.bfloat16)
    norm_w = 1 + 0.1 * torch.randn(512, generator=g)
    ang = torch.rand(cap, 32, generator=g) * 6.2831853
    positions = torch.randint(0, cap, (B,), generator=g)
    slots = torch.randperm(n_slots, generator=g)[:B]
    return kv_a, norm_w, torch.cos(ang), torch.sin(ang), positions, slots


@pytest.mark.parametrize("inter", [True, False])
@pytest.mark.parametrize("fmt,scale_fmt", [("bf16", None), ("bf16_quant", None), ("fp8", None), ("fp8", "ue8m0")])
def test_latent_append_matches_oracle(D, inter, fmt, scale_fmt):
    dev = "cuda"
    B, cap, n_slots = 9, 300, 64
    kv_a, norm_w, cos, sin, positions, slots = _latent_inputs(B, cap, n_slots, seed=17)
    slots[3] = -1  # a skipped row
    if fmt == "fp8":
        pool = torch.full((n_slots, 656), 0x55, dtype=torch.uint8, device=dev)
    else:
        pool = torch.full((n_slots, 576), 7.0, dtype=torch.bfloat16, device=dev)
    before = pool.clone()
    D.latent_append(kv_a.to(dev), norm_w.to(dev), 1e-6, cos.to(dev), sin.to(dev), positions.to(dev), slots.to(dev),
                    pool, rope_interleave=inter, fmt=fmt, scale_fmt=scale_fmt)
    torch.cuda.synchronize()
    want = O.latent_append_rows(kv_a, norm_w, 1e-6, cos, sin, positions.tolist(), inter, fmt, scale_fmt is not None)
    live = [b for b in range(B) if slots[b] >= 0]
    got = pool.cpu()[slots[live]]
    want = want[live]
    if fmt == "fp8":
        assert torch.equal(got[:, 528:], want[:, 528:])  # rope dims: the same rounded operations
        gs, ws = got[:, 512:528].contiguous().view(torch.float32), want[:, 512:528].contiguous().view(torch.float32)
        assert torch.allclose(gs, ws, rtol=2 ** -7, atol=0)
        g_lat, w_lat = O.unpack_fp8_latent(got)[:, :512].float(), O.unpack_fp8_latent(want)[:, :512].float()
        step = w_lat.abs() * 2 ** -3 + ws.repeat_interleave(128, dim=1) * 2 ** -9
        assert ((g_lat - w_lat).abs() <= step * 1.01).all()
        assert (got[:, :512] == want[:, :512]).float().mean() > 0.97
    else:
        assert torch.equal(got[:, 512:].view(torch.int16), want[:, 512:].view(torch.int16))
        g_lat, w_lat = got[:, :512].float(), want[:, :512].float()
        # RMSNorm's fp32 summation order differs from torch's: a bf16 may round the other way
        tol = 2 ** -7 if fmt == "bf16" else 2 ** -3
        assert ((g_lat - w_lat).abs() <= w_lat.abs() * tol + 1e-6).all()
        assert (got[:, :512].view(torch.int16) == want[:, :512].view(torch.int16)).float().mean() > 0.97
    untouched = torch.ones(n_slots, dtype=torch.bool)
    untouched[slots[live]] = False
    assert torch.equal(pool.cpu()[untouched].view(torch.uint8), before.cpu()[untouched].view(torch.uint8))


def test_latent_append_against_reference_fixture_and_attention(D):
    """Rows appended in the packed format are what the attention kernel reads: decode over
    them equals the oracle's decode over the reference-made rows, packed by the oracle."""
    dev = "cuda"
    g = load_golden("latent_append.npz")
    kv_a = bf16_from_bits(g["kv_a"])
    B = kv_a.shape[0]
    cos, sin = torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"])
    pool = torch.zeros(B, 576, dtype=torch.bfloat16, device=dev)
    ar = torch.arange(B)
    D.latent_append(kv_a.to(dev), torch.from_numpy(g["norm_w"]).to(dev), float(g["eps"]), cos.to(dev), sin.to(dev),
                    ar.to(dev), ar.to(dev), pool, rope_interleave=True, fmt="bf16")
    torch.cuda.synchronize()
    ref_row = torch.cat([bf16_from_bits(g["kv_norm"]), bf16_from_bits(g["k_pe"])], dim=-1)
    assert torch.equal(pool.cpu()[:, 512:].view(torch.int16), ref_row[:, 512:].view(torch.int16))
    assert ((pool.cpu()[:, :512].float() - ref_row[:, :512].float()).abs() <= ref_row[:, :512].float().abs() * 2 ** -7).all()

    # many tokens into an fp8 pool, then sparse decode over the pool
    N, H, topk = 256, 16, 128
    gen = torch.Generator().manual_seed(4)
    kv_many = (torch.randn(N, 576, generator=gen)).to(torch.bfloat16)
    ang = torch.rand(N, 32, generator=gen) * 6.2831853
    cosN, sinN = torch.cos(ang), torch.sin(ang)
    norm_w = torch.ones(512)
    pool8 = torch.zeros(1, N, 656, dtype=torch.uint8, device=dev)
    pos = torch.arange(N)
    D.latent_append(kv_many.to(dev), norm_w.to(dev), 1e-6, cosN.to(dev), sinN.to(dev), pos.to(dev), pos.to(dev),
                    pool8.view(N, 656), fmt="fp8")
    q = torch.randn(1, H, 576, generator=gen).to(torch.bfloat16)
    idx = torch.randperm(N, generator=gen)[:topk].sort().values.int().view(1, topk)
    out = D.sparse_mla_decode(q.to(dev), pool8, idx.to(dev), 192 ** -0.5)
    torch.cuda.synchronize()
    rows = O.unpack_fp8_latent(O.latent_append_rows(kv_many, norm_w, 1e-6, cosN, sinN, range(N), True, "fp8", False))
    ref = O.sparse_mla_decode(q, rows, idx, [N], 192 ** -0.5)
    assert (out.cpu().float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()
