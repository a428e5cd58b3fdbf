"""GPU tests of the serving-shaped entry (paged index keys, a slot-addressed latent
pool, per-row lengths on the device) against the CPU oracle: the reference
overlay's `_hh_fused_hide_decode_paged` contract (patch :1282-1548)."""

from __future__ import annotations

import pytest
import torch

from conftest import corr_diff, rel_err
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-2
LOGIT_TOL = 1e-2


def build_case(fp8_pool: bool, B=3, cap=2048, heads=16, hidx=64, topk=512, seed=31, lens=None, lat_rows=None):
    """lat_rows: build the latent pool from this many distinct random rows, repeated (a pool of
    two million distinct rows would only cost host time and memory)."""
    g = torch.Generator().manual_seed(seed)
    lens = [cap, 700, 1300][:B] if lens is None else list(lens)
    B = len(lens)
    pages_per = cap // 64
    num_pages = B * pages_per + 5
    perm = torch.randperm(num_pages, generator=g)[:B * pages_per].view(B, pages_per).int()
    pool_pages = torch.zeros(num_pages, 8448, dtype=torch.uint8)
    iq = torch.randn(B, hidx, 128, generator=g)
    w = torch.randn(B, hidx, generator=g) / 8
    iq8 = torch.empty(B, hidx, 128, dtype=torch.uint8)
    wp = torch.empty(B, hidx)
    ref_logits = torch.full((B, cap), float("-inf"))
    # latent rows live in one pool addressed by KV slot = page * 64 + offset
    n_slots = num_pages * 64
    lat = torch.randn(lat_rows or n_slots, 576, generator=g)
    for b in range(B):
        ik = torch.randn(cap, 128, generator=g)
        q8, k8, wf, sk = O.make_fp8_indexer_inputs(iq[b:b + 1], ik, w[b:b + 1])
        lg = O.indexer_logits_fp8(q8, k8, wf, sk)
        sk_m, _ = O.enforce_topk_margin(lg[0, :lens[b]], sk[:lens[b]], topk)
        sk = sk.clone()
        sk[:lens[b]] = sk_m.float()
        sk_full = sk
        O.pack_index_pages(k8.view(torch.uint8), sk_full, perm[b].tolist(), num_pages, pool_pages)
        iq8[b], wp[b] = q8.view(torch.uint8)[0], wf[0]
        ref_logits[b, :lens[b]] = O.indexer_logits_fp8(q8, k8[:lens[b]], wf, sk[:lens[b]])[0]
    pos2slot = (perm.long().repeat_interleave(64, dim=1) * 64 + torch.arange(64).repeat(pages_per)).int()
    kv_pool = O.pack_fp8_latent(lat) if fp8_pool else lat.to(torch.bfloat16)
    kv_ref = O.unpack_fp8_latent(kv_pool) if fp8_pool else kv_pool
    if lat_rows:  # slot s holds distinct row s % lat_rows
        kv_pool = kv_pool[torch.arange(n_slots) % lat_rows].contiguous()
    q = torch.randn(1, B, heads, 576, generator=g).to(torch.bfloat16)
    inc = torch.stack([pos2slot[b, torch.randperm(lens[b], generator=g)[:topk].sort().values.long()
                                  if lens[b] >= topk else
                                  torch.cat([torch.arange(lens[b]), torch.zeros(topk - lens[b], dtype=torch.long)])]
                       for b in range(B)]).int()
    for b in range(B):
        if lens[b] < topk:
            inc[b, lens[b]:] = -1
    inc[:, 5::37] = -1  # padding entries are skipped
    return dict(B=B, cap=cap, heads=heads, hidx=hidx, topk=topk, lens=lens, q=q, kv_pool=kv_pool, kv_ref=kv_ref,
                inc=inc, iq8=iq8, wp=wp, pages=pool_pages, pt=perm, pos2slot=pos2slot, ref_logits=ref_logits,
                lat_rows=lat_rows, n_slots=n_slots)


def call(case, **kw):
    from dsa_multi_layer_indexer_b200 import serving

    c = case
    d = lambda t: t.cuda().contiguous()
    return serving.fused_hide_decode_paged(
        d(c["q"]), d(c["kv_pool"]), d(c["inc"]), d(c["iq8"]), d(c["wp"]), d(c["pages"]), d(c["pt"]),
        d(torch.tensor(c["lens"], dtype=torch.int32)), c["cap"], 192 ** -0.5, kw.pop("pool_map", d(c["pos2slot"])), **kw)


def ref_attention(c):
    out = torch.zeros(c["B"], c["heads"], 512)
    n = c["n_slots"]
    for b in range(c["B"]):
        inc = c["inc"][b:b + 1]
        if c["lat_rows"]:  # the rows this sequence selected, gathered from the distinct ones
            live = (inc[0] >= 0) & (inc[0] < n)
            rows = c["kv_ref"][inc[0][live].long() % c["lat_rows"]]
            local = torch.full_like(inc, -1)
            local[0, live] = torch.arange(int(live.sum()), dtype=inc.dtype)
            out[b] = O.sparse_mla_decode(c["q"][0, b:b + 1], rows, local, [rows.shape[0]], 192 ** -0.5)[0]
        else:
            out[b] = O.sparse_mla_decode(c["q"][0, b:b + 1], c["kv_ref"], inc, [n], 192 ** -0.5)[0]
    return out


def ref_next(c):
    want = []
    for b in range(c["B"]):
        pos = O.select_topk(c["ref_logits"][b:b + 1], c["topk"], -1)[0]
        want.append(sorted(int(c["pos2slot"][b, p]) for p in pos.tolist() if p >= 0))
    return want


@pytest.mark.parametrize("fp8_pool", [False, True])
def test_full_mode_matches_oracle(fp8_pool):
    from dsa_multi_layer_indexer_b200 import _lib, serving

    serving.clear_scratch()
    c = build_case(fp8_pool)
    attn, nxt, logits = call(c, return_logits=True)
    assert attn.shape == (1, c["B"], c["heads"], 512) and nxt.shape == (c["B"], c["topk"]) and nxt.dtype == torch.int32
    ref = ref_attention(c)
    assert rel_err(attn[0].float().cpu(), ref) < ATTN_TOL
    assert corr_diff(attn[0].float().cpu(), ref) < 1e-3
    lg = logits.cpu()
    for b, ln in enumerate(c["lens"]):
        assert rel_err(lg[b:b + 1, :ln], c["ref_logits"][b:b + 1, :ln]) < LOGIT_TOL
        assert torch.isinf(lg[b, ln:]).all()
    got = [sorted(v for v in row if v >= 0) for row in nxt.cpu().tolist()]
    assert got == ref_next(c)  # bit-exact sets in KV-slot space
    for b, ln in enumerate(c["lens"]):
        assert (nxt[b] < 0).sum().item() == max(0, c["topk"] - ln)
    # the page-table arithmetic gives the same slots as the explicit position -> slot map
    _, nxt_pt = call(c, pool_map=None)
    assert torch.equal(nxt_pt, nxt)
    _lib.check_device_status()


def test_modes_and_select_variants():
    from dsa_multi_layer_indexer_b200 import serving

    serving.clear_scratch()
    c = build_case(True)
    attn, nxt = call(c)
    attn = attn.clone()
    nxt = nxt.clone()
    only = call(c, mode="attn_only")
    assert torch.equal(only, attn)
    slab = call(c, mode="scan_only")
    a2, lg = call(c, select=False)
    assert torch.equal(a2, attn) and torch.equal(lg, slab)
    a3, n3 = call(c, select="torch")
    assert n3.dtype == torch.int64
    for b in range(c["B"]):
        assert sorted(v for v in n3[b].tolist() if v >= 0) == sorted(v for v in nxt[b].tolist() if v >= 0)
    with pytest.raises(ValueError):
        call(c, mode="tap")
    with pytest.raises(ValueError):
        call(c, index_topk=c["topk"] // 2)


def test_head_padding_and_graph_replay():
    """20 heads are padded to 32 with zero queries and sliced off again; the call is
    capturable (no allocation after the first call, no host sync)."""
    from dsa_multi_layer_indexer_b200 import serving

    serving.clear_scratch()
    c = build_case(False, heads=20)
    attn, nxt = call(c)
    assert attn.shape == (1, c["B"], 20, 512)
    ref = ref_attention(c)
    assert rel_err(attn[0].float().cpu(), ref) < ATTN_TOL
    eager_attn, eager_nxt = attn.clone(), nxt.clone()
    d = lambda t: t.cuda().contiguous()
    args = (d(c["q"]), d(c["kv_pool"]), d(c["inc"]), d(c["iq8"]), d(c["wp"]), d(c["pages"]), d(c["pt"]),
            d(torch.tensor(c["lens"], dtype=torch.int32)), c["cap"], 192 ** -0.5, d(c["pos2slot"]))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        serving.fused_hide_decode_paged(*args)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_attn, g_nxt = serving.fused_hide_decode_paged(*args)
    g_attn.zero_()
    g_nxt.fill_(-9)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(g_attn, eager_attn) and torch.equal(g_nxt, eager_nxt)


def test_ragged_batch_at_serving_size():
    """A batch shaped like BASELINE config 4 at reduced batch (6 rows, lengths from 16384 to
    65536, page-64 index keys, fp8-packed latent pool, 128 heads, top-2048): the batch is large
    enough for the tcgen05 attention kernel; sets bit-exact, attention within 2e-2."""
    from dsa_multi_layer_indexer_b200 import _lib, serving

    serving.clear_scratch()
    lens = [65536, 16384, 40000, 23456, 65000, 32768]
    c = build_case(True, cap=65536, heads=128, topk=2048, seed=41, lens=lens)
    attn, nxt = call(c)
    ref = ref_attention(c)
    assert rel_err(attn[0].float().cpu(), ref) < ATTN_TOL
    assert corr_diff(attn[0].float().cpu(), ref) < 1e-3
    got = [sorted(v for v in row if v >= 0) for row in nxt.cpu().tolist()]
    assert got == ref_next(c)
    _lib.check_device_status()


def test_batch32_ragged_paged_fp8_at_its_full_size():
    """The batched configuration at its own size: 32 rows, lengths drawn as the benchmark draws them
    (torch.randint(16384, 65537) under seed 0), page-64 FP8 index keys behind a shuffled page table,
    FP8-packed 656-byte latent rows, 128 heads, top-2048, through the serving entry: every row's
    selected set bit-exact (scales with a margin around the cutoff), attention within 2e-2."""
    from dsa_multi_layer_indexer_b200 import _lib, serving

    serving.clear_scratch()
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16384, 65537, (32,), generator=g, dtype=torch.int32).tolist()
    c = build_case(True, cap=65536, heads=128, topk=2048, seed=44, lens=lens, lat_rows=1 << 16)
    attn, nxt, logits = call(c, return_logits=True)
    torch.cuda.synchronize()
    _lib.check_device_status()
    lg = logits.cpu()
    for b, ln in enumerate(lens):
        assert rel_err(lg[b:b + 1, :ln], c["ref_logits"][b:b + 1, :ln]) < LOGIT_TOL
        assert torch.isinf(lg[b, ln:]).all()
    got = [sorted(v for v in row if v >= 0) for row in nxt.cpu().tolist()]
    assert got == ref_next(c)
    ref = ref_attention(c)
    assert rel_err(attn[0].float().cpu(), ref) < ATTN_TOL
    assert corr_diff(attn[0].float().cpu(), ref) < 1e-3
    serving.clear_scratch()


def test_forward_hide_operands_stages_and_feeds_the_paged_scan():
    """A few decode steps through the overlay-shaped operand hook (prepare + store,
    no top-k), then the paged scan over what it stored, against the oracle's staging
    and logits (patch :252-363 + :1282-1548 in the reference)."""
    from dsa_multi_layer_indexer_b200 import serving

    dev = "cuda"
    B, H, pages_per, T = 3, 64, 3, 150
    cap = pages_per * 64
    g = torch.Generator().manual_seed(5)
    num_pages = B * pages_per + 2
    perm = torch.randperm(num_pages, generator=g)[: B * pages_per].view(B, pages_per).to(torch.int32)
    pages = torch.zeros(num_pages, 8448, dtype=torch.uint8, device=dev)
    ang = torch.rand(cap, 32, generator=g) * 6.2831853
    cos, sin = torch.cos(ang), torch.sin(ang)
    norm_w, norm_b = 1 + 0.1 * torch.randn(128, generator=g), 0.05 * torch.randn(128, generator=g)
    o_k = torch.zeros(B, cap, 128, dtype=torch.uint8)
    o_s = torch.zeros(B, cap)
    lens = torch.zeros(B, dtype=torch.int32, device=dev)
    ptrs = set()
    for t in range(T):
        q_proj = torch.randn(B, H, 128, generator=g).to(torch.bfloat16)
        k_proj = torch.randn(B, 128, generator=g).to(torch.bfloat16)
        gates = torch.randn(B, H, generator=g)
        positions = torch.full((B,), t, dtype=torch.int64)
        lens.fill_(t + 1)
        ret = serving.forward_hide_operands(q_proj.to(dev), k_proj.to(dev), gates.to(dev), norm_w.to(dev),
                                            norm_b.to(dev), 1e-6, cos.to(dev), sin.to(dev), positions.to(dev),
                                            pages, perm.to(dev), lens)
        q_fp8, weights, pg, pt, sl, skv_cap = ret
        ptrs.add((q_fp8.data_ptr(), weights.data_ptr()))
        q8, w, k8, ks = O.indexer_stage_fp8(q_proj, k_proj, gates, norm_w, norm_b, 1e-6, cos, sin, [t] * B,
                                            False, False, 128 ** -0.5)
        o_k[:, t], o_s[:, t] = k8, ks
    assert len(ptrs) == 1 and skv_cap == cap and pt.dtype == torch.int32 and sl.dtype == torch.int32
    assert q_fp8.shape == (B, H, 128) and weights.shape == (B, H) and pg.data_ptr() == pages.data_ptr()
    assert torch.equal(q_fp8.cpu(), q8) and torch.equal(weights.cpu(), w)
    logits = serving.fused_hide_decode_paged(
        torch.zeros(1, B, 128, 576, dtype=torch.bfloat16, device=dev), torch.zeros(64, 576, dtype=torch.bfloat16, device=dev),
        torch.full((B, 2048), -1, dtype=torch.int32, device=dev), q_fp8, weights, pages, pt, sl, skv_cap,
        192 ** -0.5, None, index_topk=2048, mode="scan_only")
    torch.cuda.synchronize()
    for b in range(B):
        ref = O.indexer_logits_fp8(q8[b:b + 1], o_k[b, :T], w[b:b + 1], o_s[b, :T])[0]
        got = logits[b, :T].cpu()
        assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()
        assert torch.isinf(logits[b, T:].cpu()).all()
    with pytest.raises(RuntimeError, match="HIDE VOID"):
        serving.forward_hide_operands(q_proj.to(dev), k_proj.to(dev), gates.to(dev), norm_w.to(dev), norm_b.to(dev),
                                      1e-6, cos.to(dev), sin.to(dev), positions.to(dev),
                                      torch.zeros(4, 4224, dtype=torch.uint8, device=dev), perm.to(dev), lens)
