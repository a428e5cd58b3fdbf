"""GPU parity tests: every kernel, called through the C ABI, against the CPU
oracle on the same seeded inputs and against the reference-generated golden
fixtures. Tolerances are the ones the task states: index sets bit-exact,
indexer logits <= 1e-2 relative, attention output <= 2e-2 relative (bf16), with
"relative" = max|a-b| / max|b| as the reference measures it."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, corr_diff, load_golden, rel_err
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-2
ATTN_TOL = 2e-2


@pytest.fixture(scope="module")
def ops():
    from dsa_multi_layer_indexer_b200 import _lib, ops as _ops

    _lib.lib()  # fail loudly if the library is missing
    yield _ops
    _lib.check_device_status()


def dev(t: torch.Tensor) -> torch.Tensor:
    return t.cuda().contiguous()


def make_indexer(seed, rows, n_heads, n_keys):
    g = torch.Generator().manual_seed(seed)
    iq = torch.randn(rows, n_heads, 128, generator=g)
    ik = torch.randn(n_keys, 128, generator=g)
    w = torch.randn(rows, n_heads, generator=g) / 8
    return O.make_fp8_indexer_inputs(iq, ik, w)


# ----------------------------------------------------------------------------- scan
@pytest.mark.parametrize("impl", [0, 1])
def test_scan_golden(ops, impl):
    g = load_golden("indexer_fp8.npz")
    iq8, ik8, wp, sk = (torch.from_numpy(g[k]) for k in ("iq8", "ik8", "wp", "sk"))
    got = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), rows_per_seq=2, impl=impl)
    ref = torch.from_numpy(g["logits"])
    assert rel_err(got.cpu(), ref) < 1e-5
    assert corr_diff(got.cpu(), ref) < 1e-9


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("n_keys,n_heads", [(1, 64), (127, 64), (128, 16), (129, 32), (1000, 64), (4096, 64), (5000, 48)])
def test_scan_shapes(ops, impl, n_keys, n_heads):
    iq8, ik8, wp, sk = make_indexer(n_keys, 1, n_heads, n_keys)
    got = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), impl=impl)
    ref = O.indexer_logits_fp8(iq8, ik8, wp, sk)
    assert got.shape == ref.shape
    assert rel_err(got.cpu(), ref) < 1e-5


def test_scan_ragged_batch_and_mask(ops):
    B, cap = 5, 1500
    lens = [1500, 1, 129, 640, 0]
    torch.manual_seed(3)
    iq = torch.randn(B, 64, 128)
    ik = torch.randn(B, cap, 128)
    w = torch.randn(B, 64) / 8
    iq8, sq = O.quantize_e4m3_rowwise(iq)
    ik8, sk = O.quantize_e4m3_rowwise(ik)
    wp = sq * w
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    out = torch.full((B, 1504), 7.0, device="cuda")
    got = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), dev(seq_lens), out=out).cpu()
    for b in range(B):
        ref = O.indexer_logits_fp8(iq8[b:b + 1], ik8[b], wp[b:b + 1], sk[b])[0]
        n = lens[b]
        if n:
            assert rel_err(got[b, :n], ref[:n]) < 1e-5
        assert torch.isinf(got[b, n:]).all() and (got[b, n:] < 0).all()
    assert (out[:, 1500:] == 7.0).all()  # columns past ctx are not written


def test_scan_ragged_batch_of_32_rows_on_the_shared_out_grid(ops):
    """32 rows of very different lengths (empty ones among them) on the 1-D grid whose CTAs are
    shared out by tile count; an output slab whose rows are not 16-byte aligned (the dead tail is
    then filled by scalar stores); the per-row histogram counts exactly the visible logits."""
    B, cap, stride = 32, 3000, 3001
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(0, cap + 1, (B,), generator=g).tolist()
    lens[0], lens[5], lens[31] = 0, cap, 1
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, 64, 128, generator=g))
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, cap, 128, generator=g))
    wp = sq * (torch.randn(B, 64, generator=g) / 8)
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    out = torch.full((B, stride), 7.0, device="cuda")
    hist = torch.zeros(B, ops.HIST_BINS, dtype=torch.int32, device="cuda")
    got = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), dev(seq_lens), out=out, hist=hist).cpu()
    hist = hist.cpu()
    for b in range(B):
        n = lens[b]
        if n:
            ref = O.indexer_logits_fp8(iq8[b:b + 1], ik8[b], wp[b:b + 1], sk[b])[0]
            assert rel_err(got[b, :n], ref[:n]) < 1e-5, b
        assert torch.isinf(got[b, n:cap]).all() and (got[b, n:cap] < 0).all(), b
        bits = got[b, :n].contiguous().view(torch.int32).long() & 0xFFFFFFFF
        key = torch.where(bits >> 31 != 0, ~bits & 0xFFFFFFFF, bits | 0x80000000)
        assert torch.equal(hist[b].long(), torch.bincount(key >> 20, minlength=ops.HIST_BINS)), b
    assert (out[:, cap:] == 7.0).all()  # columns past ctx are not written


def test_scan_full_context_128k(ops):
    n = 131072
    iq8, ik8, wp, sk = make_indexer(0, 1, 64, n)
    got = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk)).cpu()
    ref = O.indexer_logits_fp8(iq8, ik8, wp, sk)
    assert rel_err(got, ref) < 1e-5
    legacy = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), impl=1).cpu()
    assert rel_err(legacy, ref) < 1e-5


def test_scan_paged_equals_dense(ops):
    B, cap = 3, 1024
    lens = [1000, 64, 513]
    torch.manual_seed(5)
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, 64, 128))
    wp = sq * (torch.randn(B, 64) / 8)
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, cap, 128))
    pages_per = cap // 64
    num_pages = B * pages_per + 3
    perm = torch.randperm(num_pages)[: B * pages_per].reshape(B, pages_per)
    pool = torch.zeros(num_pages, 8448, dtype=torch.uint8)
    for b in range(B):
        O.pack_index_pages(ik8[b], sk[b], perm[b].tolist(), num_pages, pool)
    seq_lens = dev(torch.tensor(lens, dtype=torch.int32))
    dense = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), seq_lens).cpu()
    paged = ops.indexer_scan_fp8_paged(dev(iq8), dev(wp), dev(pool), dev(perm.int()), seq_lens, cap).cpu()
    assert torch.equal(dense, paged)


def test_scan_f32_matches_oracle(ops):
    torch.manual_seed(0)
    B, S, H, D = 2, 12, 8, 16
    q, k, w = torch.randn(B, S, H, D), torch.randn(B, S, D), torch.randn(B, S, H)
    lens = torch.arange(1, S + 1, dtype=torch.int32).repeat(B)
    got = ops.indexer_scan_f32(dev(q.reshape(B * S, H, D)), dev(w.reshape(B * S, H)), dev(k), dev(lens),
                               rows_per_seq=S).cpu().reshape(B, S, S)
    ref = O.indexer_logits_f32(q, k, w)
    for b in range(B):
        masked = O.mask_beyond(ref[b], list(range(1, S + 1)))
        fin = torch.isfinite(masked)
        assert torch.equal(torch.isfinite(got[b]), fin)
        assert torch.allclose(got[b][fin], masked[fin], rtol=1e-5, atol=1e-5)


# ----------------------------------------------------------------------------- top-k
def check_topk(ops, logits, topk, lens=None, pad=-1):
    R, n = logits.shape
    seq = None if lens is None else dev(torch.tensor(lens, dtype=torch.int32))
    got, vals = ops.topk_select(dev(logits), topk, seq, pad_value=pad, return_values=True)
    got, vals = got.cpu(), vals.cpu()
    masked = logits if lens is None else O.mask_beyond(logits, lens)
    ref = O.select_topk(masked, topk, pad_value=pad)
    assert torch.equal(got.long(), ref), "selected index set / order differs from the oracle"
    for r in range(R):
        keep = got[r] >= 0
        assert torch.equal(vals[r][keep], logits[r][got[r][keep].long()])


@pytest.mark.parametrize("n,topk", [(100, 16), (2048, 2048), (4096, 2048), (5000, 64), (32768, 2048),
                                    (40000, 2048), (131072, 2048), (131073, 2048), (200000, 2048), (262144, 2048),
                                    (262145, 2048), (1 << 20, 4096)])
def test_topk_random(ops, n, topk):
    torch.manual_seed(n)
    check_topk(ops, torch.randn(2, n), topk)


def test_topk_heavy_ties_pick_lower_positions(ops):
    torch.manual_seed(1)
    n = 50000
    coarse = torch.randint(-8, 8, (3, n)).float() * 0.25  # 16 distinct values: thousands of ties at the cutoff
    check_topk(ops, coarse, 2048)
    check_topk(ops, torch.zeros(1, n), 2048)
    check_topk(ops, -torch.ones(1, 9000), 100)


def test_topk_short_rows_and_neg_inf(ops):
    torch.manual_seed(2)
    logits = torch.randn(4, 6000)
    check_topk(ops, logits, 2048, lens=[6000, 2048, 100, 0])
    logits[0, 10:5990] = float("-inf")  # fewer finite entries than k: the rest is padding
    got = ops.topk_select(dev(logits[:1]), 64, pad_value=-1).cpu()[0]
    ref = O.select_topk(logits[:1], 64, pad_value=-1)[0]
    assert sorted(got[got >= 0].tolist()) == sorted(ref[ref >= 0].tolist())
    assert int((got < 0).sum()) == 64 - 20


def test_topk_mixed_rows_repeated(ops):
    """Twelve rows of one launch that take every path of the cluster kernel (random, heavy ties,
    all equal, sorted so that the candidates sit in one CTA, short and boundary lengths), with and
    without the 12-bit histogram, against a stable descending sort; the launch is then replayed
    500 times from a graph and every result compared (a race between CTAs would show as a rare miss)."""
    torch.manual_seed(1)
    R, n, topk = 12, 60000, 2048
    logits = torch.randn(R, n, device="cuda") * 5
    logits[1] = torch.randint(0, 40, (n,), device="cuda").float()
    logits[2] = torch.randint(0, 3, (n,), device="cuda").float()
    logits[3] = 1.0
    logits[4, ::3] = logits[4, 0]
    logits[5] = torch.sort(logits[5]).values
    lens = torch.tensor([n, n, n, n, n, n, 100, 2048, 2049, 30000, 16384, 16385], dtype=torch.int32, device="cuda")

    def reference(row, ln):
        order = torch.sort(row[:ln], descending=True, stable=True).indices[:topk]
        out = torch.full((topk,), -1, dtype=torch.int32, device="cuda")
        out[:order.numel()] = torch.sort(order).values.int()
        return out

    want = torch.stack([reference(logits[r], int(lens[r])) for r in range(R)])
    key = logits.view(torch.int32)
    bins = ((torch.where(key < 0, ~key, key | -2147483648) >> 20) & 0xFFF).long()
    hist0 = torch.stack([torch.bincount(bins[r, :int(lens[r])], minlength=ops.HIST_BINS) for r in range(R)]).int()
    for use_hist in (False, True):
        hist = hist0.clone() if use_hist else None
        out = torch.empty(R, topk, dtype=torch.int32, device="cuda")
        ops.topk_select(logits, topk, lens, hist=hist, out_idx=out)
        assert torch.equal(out, want), use_hist
        if use_hist:
            assert int(hist.abs().sum()) == 0  # consumed and re-armed
            hist.copy_(hist0)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph):
                ops.topk_select(logits, topk, lens, hist=hist, out_idx=out)
                if use_hist:
                    hist.copy_(hist0)
        torch.cuda.current_stream().wait_stream(side)
        bad = torch.zeros((), dtype=torch.int64, device="cuda")
        for _ in range(500):
            graph.replay()
            bad += (out != want).any()
        assert int(bad) == 0, use_hist


def test_topk_strided_slab_offset_and_map(ops):
    torch.manual_seed(4)
    slab = torch.randn(3, 8192)
    view = dev(slab)[:, :7000]
    got = ops.topk_select(view, 512, index_offset=1000).cpu()
    ref = O.select_topk(slab[:, :7000], 512, pad_value=-1) + 1000
    assert torch.equal(got.long(), ref)
    imap = torch.randint(0, 1 << 20, (3, 7000), dtype=torch.int32)
    got = ops.topk_select(view, 512, index_map=dev(imap)).cpu()
    ref = O.select_topk(slab[:, :7000], 512, pad_value=-1)
    assert torch.equal(got.long(), torch.gather(imap.long(), 1, ref))


def test_topk_with_scan_histogram_equals_plain(ops):
    n = 20000
    B = 3
    lens = [20000, 7777, 2500]
    torch.manual_seed(9)
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, 64, 128))
    wp = sq * (torch.randn(B, 64) / 8)
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, n, 128))
    seq_lens = dev(torch.tensor(lens, dtype=torch.int32))
    for impl in (0, 1):
        hist = torch.zeros(B, 4096, dtype=torch.int32, device="cuda")
        logits = ops.indexer_scan_fp8(dev(iq8), dev(wp), dev(ik8), dev(sk), seq_lens, hist=hist, impl=impl)
        assert hist.sum(1).cpu().tolist() == lens
        plain = ops.topk_select(logits, 2048, seq_lens)
        fused = ops.topk_select(logits, 2048, seq_lens, hist=hist)
        assert torch.equal(plain, fused)
        assert int(hist.abs().sum()) == 0  # re-armed for the next launch


def test_topk_and_paged_scan_wrappers_reject_buffers_of_the_wrong_extent(ops):
    """The wrappers hand raw pointers to the kernels, so every caller-owned output is checked
    for device, dtype and extent first: a short or host buffer is a ValueError, not a wild write."""
    logits = torch.randn(2, 5000, device="cuda")
    with pytest.raises(ValueError, match="out_idx"):
        ops.topk_select(logits, 64, out_idx=torch.empty(2, 32, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError, match="out_val"):
        ops.topk_select(logits, 64, out_val=torch.empty(2, 64))  # host memory
    with pytest.raises(ValueError, match="out_val"):
        ops.topk_select(logits, 64, out_val=torch.empty(2, 63, device="cuda"))
    with pytest.raises(ValueError, match="hist"):
        ops.topk_select(logits, 64, hist=torch.zeros(1, 4096, dtype=torch.int32, device="cuda"))
    iq = torch.zeros(2, 64, 128, dtype=torch.uint8, device="cuda")
    w = torch.zeros(2, 64, device="cuda")
    pool = torch.zeros(8, 8448, dtype=torch.uint8, device="cuda")
    pt = torch.zeros(2, 4, dtype=torch.int32, device="cuda")
    lens = torch.full((2,), 256, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="out must be"):
        ops.indexer_scan_fp8_paged(iq, w, pool, pt, lens, 256, out=torch.empty(2, 128, device="cuda"))
    with pytest.raises(ValueError, match="out must be"):
        ops.indexer_scan_fp8_paged(iq, w, pool, pt, lens, 256, out=torch.empty(1, 256, device="cuda"))
    with pytest.raises(ValueError, match="cannot cover"):
        ops.indexer_scan_fp8_paged(iq, w, pool, pt, lens, 512)


# ----------------------------------------------------------------------------- sparse MLA
def test_sparse_mla_golden(ops):
    g = load_golden("sparse_mla.npz")
    q = bf16_from_bits(g["q"])[0]
    kv = bf16_from_bits(g["kv"])[0, :, 0]
    idx = torch.from_numpy(g["indices"])
    S, N = q.shape[0], kv.shape[0]
    lens = torch.tensor([(N - S) + s + 1 for s in range(S)], dtype=torch.int32)
    for nsplit in (1, 2, 4):
        got = ops.sparse_mla_decode(dev(q), dev(kv), dev(idx), float(g["sm_scale"]), dev(lens),
                                    rows_per_seq=S, nsplit=nsplit).float().cpu()
        ref = torch.from_numpy(g["out"])[0]
        assert rel_err(got, ref) < ATTN_TOL
        assert corr_diff(got, ref) < 1e-3


@pytest.mark.parametrize("H,topk,n,nsplit", [(16, 64, 300, 1), (16, 2048, 4096, 32), (128, 2048, 8192, 32),
                                             (32, 2048, 3000, 7), (64, 512, 2000, 8), (16, 80, 100, 3)])
def test_sparse_mla_random(ops, H, topk, n, nsplit):
    torch.manual_seed(H + topk)
    q = torch.randn(1, H, 576).to(torch.bfloat16)
    kv = torch.randn(n, 576).to(torch.bfloat16)
    idx = torch.full((1, topk), -1, dtype=torch.int32)
    take = min(topk, n)
    idx[0, :take] = torch.randperm(n)[:take].int()
    idx[0, ::17] = n + 5  # entries beyond the sequence are skipped
    sm = 192 ** -0.5
    got = ops.sparse_mla_decode(dev(q), dev(kv), dev(idx), sm, nsplit=nsplit).float().cpu()
    ref = O.sparse_mla_decode(q, kv, idx, [n], sm)
    assert rel_err(got, ref) < ATTN_TOL
    assert corr_diff(got, ref) < 1e-3


def test_sparse_mla_batched_equals_rows_bitwise(ops):
    torch.manual_seed(11)
    B, H, n, topk = 4, 32, 2500, 1024
    q = torch.randn(B, H, 576).to(torch.bfloat16)
    kv = torch.randn(B, n, 576).to(torch.bfloat16)
    lens = [2500, 1, 1300, 64]
    idx = torch.stack([torch.randperm(n)[:topk] for _ in range(B)]).int()
    seq = dev(torch.tensor(lens, dtype=torch.int32))
    sm = 576 ** -0.5
    both = ops.sparse_mla_decode(dev(q), dev(kv), dev(idx), sm, seq, nsplit=8).cpu()
    for b in range(B):
        one = ops.sparse_mla_decode(dev(q[b:b + 1]), dev(kv[b:b + 1]), dev(idx[b:b + 1]), sm, seq[b:b + 1],
                                    nsplit=8).cpu()
        assert torch.equal(one[0], both[b])
        ref = O.sparse_mla_decode(q[b:b + 1], kv[b], idx[b:b + 1], [lens[b]], sm)
        assert rel_err(both[b:b + 1].float(), ref) < ATTN_TOL


def test_sparse_mla_dense_cold_start(ops):
    torch.manual_seed(12)
    H, n = 16, 700
    q = torch.randn(1, H, 576).to(torch.bfloat16)
    kv = torch.randn(n, 576).to(torch.bfloat16)
    seq = dev(torch.tensor([650], dtype=torch.int32))
    got = ops.sparse_mla_decode(dev(q), dev(kv), None, 0.07, seq, nsplit=4).float().cpu()
    ref = O.dense_mla_decode(q, kv, [650], 0.07)
    assert rel_err(got, ref) < ATTN_TOL


def test_sparse_mla_fp8_latent_rows(ops):
    torch.manual_seed(13)
    H, n, topk = 32, 3000, 2048
    q = torch.randn(1, H, 576).to(torch.bfloat16)
    rows = O.pack_fp8_latent(torch.randn(n, 576))
    idx = torch.randperm(n)[:topk].int().unsqueeze(0)
    sm = 192 ** -0.5
    got = ops.sparse_mla_decode(dev(q), dev(rows), dev(idx), sm, nsplit=16).float().cpu()
    ref = O.sparse_mla_decode(q, O.unpack_fp8_latent(rows), idx, [n], sm)
    assert rel_err(got, ref) < ATTN_TOL
    assert corr_diff(got, ref) < 1e-3


def test_sparse_mla_f32_matches_oracle(ops):
    g = load_golden("attention_core_f32.npz")
    mq, mkv = torch.from_numpy(g["mq"]), torch.from_numpy(g["mkv"])
    idx = torch.from_numpy(g["idx"])
    B, S, H, D = mq.shape
    lens = dev(torch.arange(1, S + 1, dtype=torch.int32).repeat(B))
    sm = D ** -0.5
    sp = ops.sparse_mla_f32(dev(mq.reshape(B * S, H, D)), dev(mkv), dev(idx.reshape(B * S, -1).int()), 64, sm,
                            lens, rows_per_seq=S).cpu().reshape(B, S, H, 64)
    assert torch.allclose(sp, torch.from_numpy(g["sparse"]), rtol=1e-4, atol=1e-5)
    de = ops.sparse_mla_f32(dev(mq.reshape(B * S, H, D)), dev(mkv), None, 64, sm, lens,
                            rows_per_seq=S).cpu().reshape(B, S, H, 64)
    assert torch.allclose(de, torch.from_numpy(g["dense"]), rtol=1e-4, atol=1e-5)


# ----------------------------------------------------------------------------- quantiser, errors
def test_quantiser_bit_exact(ops):
    g = load_golden("fp8_formats.npz")
    q, s = ops.quantize_e4m3_rowwise(dev(torch.from_numpy(g["x"])))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g["xq"])
    assert np.array_equal(s.cpu().numpy(), g["xs"])


def test_bad_arguments_raise(ops):
    from dsa_multi_layer_indexer_b200._lib import DsaError

    iq8, ik8, wp, sk = make_indexer(0, 1, 64, 256)
    with pytest.raises(DsaError):
        ops.indexer_scan_fp8(dev(iq8[:, :24]), dev(wp[:, :24]), dev(ik8), dev(sk))  # heads not a multiple of 16
    with pytest.raises(ValueError):
        ops.sparse_mla_decode(torch.zeros(1, 8, 576, dtype=torch.bfloat16, device="cuda"),
                              torch.zeros(10, 576, dtype=torch.bfloat16, device="cuda"), None, 1.0)
    with pytest.raises(DsaError):
        ops.topk_select(torch.zeros(1, (1 << 20) + 1, device="cuda"), 2048)


# ----------------------------------------------------------------------------- fused launch
@pytest.mark.parametrize("B,H,n,topk,nsplit", [(1, 128, 20000, 2048, 32), (3, 32, 5000, 1024, 8), (2, 16, 700, 64, 1)])
def test_fused_indexer_attention_launch_equals_separate_launches(ops, B, H, n, topk, nsplit):
    """One role-split launch (attention over a given selection + the indexer scan)
    returns bit for bit what the two separate launches return (the role-split launch
    contains the mma.sync attention body; at these sizes the separate launch takes it too)."""
    torch.manual_seed(B * 1000 + H)
    q = dev(torch.randn(B, H, 576).to(torch.bfloat16))
    kv = dev(torch.randn(B, n, 576).to(torch.bfloat16))
    attend = dev(torch.stack([torch.randperm(n)[:topk] for _ in range(B)]).int())
    iq8, sq = O.quantize_e4m3_rowwise(torch.randn(B, 64, 128))
    ik8, sk = O.quantize_e4m3_rowwise(torch.randn(B, n, 128))
    wp = dev(sq * (torch.randn(B, 64) / 8))
    iq8, ik8, sk = dev(iq8), dev(ik8), dev(sk)
    lens = dev(torch.randint(max(1, n // 2), n + 1, (B,), dtype=torch.int32))
    sm = 192 ** -0.5
    hist_a = torch.zeros(B, 4096, dtype=torch.int32, device="cuda")
    hist_b = torch.zeros(B, 4096, dtype=torch.int32, device="cuda")
    out_f, logits_f = ops.fused_decode(q, kv, attend, sm, iq8, wp, ik8, sk, lens, nsplit=nsplit, hist=hist_a)
    from dsa_multi_layer_indexer_b200 import ops as _o
    scratch = _o.MlaScratch(B, H, nsplit, "cuda")
    out_s = ops.sparse_mla_decode(q, kv, attend, sm, lens, nsplit=nsplit, scratch=scratch)
    logits_s = ops.indexer_scan_fp8(iq8, wp, ik8, sk, lens, hist=hist_b)
    assert torch.equal(out_f, out_s)
    assert torch.equal(logits_f, logits_s)
    assert torch.equal(hist_a, hist_b)
    sel = ops.topk_select(logits_f, topk, lens, hist=hist_a)
    assert torch.equal(sel, ops.topk_select(logits_s, topk, lens))


def test_a_wait_that_runs_out_reports_and_clears(ops):
    """Every wait in the library's kernels is bounded. One CTA waits 1 ms on a barrier that
    nothing completes: the kernel returns, the status call reports the time-out once, and the
    word is clear again afterwards (nothing faults or hangs; the context stays usable)."""
    from dsa_multi_layer_indexer_b200 import _lib

    torch.cuda.synchronize()
    _lib.check_device_status()
    _lib.check(_lib.lib().dsa_debug_wait_timeout(1_000_000, torch.cuda.current_stream().cuda_stream))
    with pytest.raises(_lib.DsaError) as err:
        _lib.check_device_status()
    assert err.value.status == -4  # DSA_ERR_DEVICE_TIMEOUT
    _lib.check_device_status()  # cleared
    with pytest.raises(_lib.DsaError):  # the limit is capped at 10 ms
        _lib.check(_lib.lib().dsa_debug_wait_timeout(10_000_001, torch.cuda.current_stream().cuda_stream))
    x = torch.arange(8, device="cuda").sum().item()  # the context still works
    assert x == 28
