"""GPU tests of the decode-time driver: the persistent-buffer step, its CUDA
graph, and the host-buffer form whose copies are nodes of the same graph and
whose attention output is written straight into pinned host memory."""

from __future__ import annotations

import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


def make_case(ctx=8192, heads=32, index_heads=64, topk=2048, seed=5):
    from dsa_multi_layer_indexer_b200 import ops
    from dsa_multi_layer_indexer_b200.decode import HotPathState, LayerCache

    g = torch.Generator().manual_seed(seed)
    iq = torch.randn(1, index_heads, 128, generator=g)
    ik = torch.randn(ctx, 128, generator=g)
    w = torch.randn(1, index_heads, generator=g) / 8
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(iq, ik, w)
    q = torch.randn(1, heads, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(1, ctx, 576, generator=g).to(torch.bfloat16)
    cache = LayerCache(ik8.view(torch.uint8).view(1, ctx, 128).cuda(), sk.view(1, ctx).cuda(), kv.cuda())
    st = HotPathState(1, heads, index_heads, ctx, topk, "cuda")
    host = dict(iq8=iq8.view(torch.uint8).view(1, index_heads, 128), w=wp.view(1, index_heads), q=q)
    st.index_q.copy_(host["iq8"])
    st.index_w.copy_(host["w"])
    st.q.copy_(q)
    st.seq_lens.fill_(ctx - 3)
    return ops, st, cache, host


def test_step_graph_and_host_decoder_agree():
    from dsa_multi_layer_indexer_b200 import _lib
    from dsa_multi_layer_indexer_b200.decode import HostDecoder

    ops, st, cache, host = make_case()
    sm = 192 ** -0.5
    eager = st.run(cache, sm).clone()
    idx_eager = st.indices.clone()
    # the three launches, called one by one through ops, give the same answer
    logits = ops.indexer_scan_fp8(st.index_q, st.index_w, cache.index_k, cache.k_scale, st.seq_lens, ctx=st.capacity)
    idx = ops.topk_select(logits, st.topk, st.seq_lens)
    assert torch.equal(idx, idx_eager)
    out = ops.sparse_mla_decode(st.q, cache.kv, idx, sm, st.seq_lens, nsplit=st.nsplit)
    assert torch.equal(out, eager)
    # captured graph
    graph = st.capture(cache, sm)
    st.out.zero_()
    st.indices.fill_(-7)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(st.out, eager) and torch.equal(st.indices, idx_eager)
    # host buffers in, host buffers out, twice in a row
    dec = HostDecoder(st, cache, sm)
    dec.h_index_q.copy_(host["iq8"])
    dec.h_index_w.copy_(host["w"])
    dec.h_q.copy_(host["q"])
    for _ in range(2):
        st.in_arena.zero_()  # the step must bring its own inputs
        dec.h_out.zero_()
        dec.h_indices.fill_(-7)
        got = dec.step()
        assert not got.is_cuda
        assert torch.equal(got, eager.cpu())
        assert torch.equal(dec.h_indices, idx_eager.cpu())
    assert dec.h2d_bytes == st.in_arena.numel() and dec.d2h_bytes == st.out_arena.numel()
    _lib.check_device_status()


def test_copy_bytes_between_pinned_host_and_device():
    from dsa_multi_layer_indexer_b200 import ops

    src = torch.arange(4096, dtype=torch.int32).pin_memory()
    dst = torch.zeros(4096, dtype=torch.int32, device="cuda")
    ops.copy_bytes(dst, src)
    back = torch.zeros(4096, dtype=torch.int32).pin_memory()
    ops.copy_bytes(back, dst)
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), src) and torch.equal(back, src)
    with pytest.raises(ValueError):
        ops.copy_bytes(dst[:3], src[:3])  # 12 bytes: not a multiple of 16
    with pytest.raises(ValueError):
        ops.copy_bytes(dst, torch.zeros(4096, dtype=torch.int32))  # pageable host memory


def test_copy_beside_the_previous_kernel_and_copy_with_epoch():
    """The copy that runs beside the kernel enqueued before it completes after that kernel, and
    the next launch sees both: a top-k, then a copy from pinned memory beside it, then a kernel
    copy that reads what the two wrote. The final node copies and posts the epoch word in one launch."""
    from dsa_multi_layer_indexer_b200 import ops

    torch.manual_seed(3)
    n = 65536
    src = torch.empty(36864, dtype=torch.int32).pin_memory()
    dst = torch.zeros(36864, dtype=torch.int32, device="cuda")
    sel = torch.empty(1, 2048, dtype=torch.int32, device="cuda")
    seen = torch.zeros(36864 + 2048, dtype=torch.int32, device="cuda")
    back = torch.zeros(36864 + 2048, dtype=torch.int32).pin_memory()
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    for it in range(20):
        logits = torch.randn(1, n, device="cuda")
        src.copy_(torch.randint(0, 1 << 30, (36864,), dtype=torch.int32))
        ops.topk_select(logits, 2048, out_idx=sel)
        ops.copy_bytes(dst, src, beside_previous=True)
        ops.copy_bytes(seen[:36864], dst)
        ops.copy_bytes(seen[36864:], sel.view(-1))
        ops.copy_post_epoch(back, seen, counter, flag)
        torch.cuda.synchronize()
        assert int(flag.item()) == it + 1
        assert torch.equal(back[:36864], src)
        want = torch.topk(logits[0], 2048).indices.sort().values.int().cpu()
        assert torch.equal(back[36864:].sort().values, want)
    with pytest.raises(ValueError):
        ops.copy_post_epoch(back[:3], seen[:3], counter, flag)


def test_lagged_layer_as_one_chain_equals_the_separate_launches():
    """The lagged layer on one stream (scan, top-k, then the attention over the PREVIOUS selection
    enqueued behind the top-k and running beside it) returns bit for bit what the indexer and
    the attention return when they are launched one after the other, eagerly and from a graph,
    and what is enqueued after the chain sees the top-k's selection as well as the attention's output."""
    from dsa_multi_layer_indexer_b200 import _lib

    ops, st, cache, host = make_case(ctx=20000, heads=32, topk=1024, seed=9)
    sm = 192 ** -0.5
    st.index_q.copy_(host["iq8"])
    st.index_w.copy_(host["w"])
    st.q.copy_(host["q"])
    torch.manual_seed(4)
    attend = torch.stack([torch.randperm(20000)[:1024] for _ in range(st.rows)]).int().cuda()
    st.run_indexer(cache)
    sel_ref = st.indices.clone()
    out_ref = st.run_attention(cache, attend, sm).clone()
    for _ in range(3):
        st.indices.fill_(-1)
        st.out.zero_()
        st.run_lagged_chained(cache, attend, sm)
        both = torch.cat([st.indices.view(-1), st.out.view(torch.int16).view(-1).int()])  # enqueued after the chain
        torch.cuda.synchronize()
        assert torch.equal(st.indices, sel_ref) and torch.equal(st.out, out_ref)
        assert torch.equal(both[:sel_ref.numel()], sel_ref.view(-1))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        st.run_lagged_chained(cache, attend, sm)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(4):
            st.run_lagged_chained(cache, attend, sm)
    for _ in range(3):
        st.indices.fill_(-1)
        st.out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(st.indices, sel_ref) and torch.equal(st.out, out_ref)
    _lib.check_device_status()


def test_host_decoder_stream_sync_mode_agrees_with_polling():
    from dsa_multi_layer_indexer_b200.decode import HostDecoder

    ops, st, cache, host = make_case(ctx=4096, heads=16, topk=512, seed=6)
    sm = 192 ** -0.5
    outs = []
    for kw in (dict(poll=True, kernel_copies=True), dict(poll=False, kernel_copies=False)):
        dec = HostDecoder(st, cache, sm, **kw)
        dec.h_index_q.copy_(host["iq8"])
        dec.h_index_w.copy_(host["w"])
        dec.h_q.copy_(host["q"])
        for _ in range(3):
            dec.h_out.zero_()
            got = dec.step().clone()
        outs.append((got, dec.h_indices.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert float(outs[0][0].float().abs().max()) > 0


def test_hot_path_at_config2_size_matches_oracle():
    """BASELINE config 2 at full size (batch 1, context 131072, 64 x 128 FP8 indexer,
    top-2048, 128 MLA heads bf16) through the persistent-buffer step: logits within
    1e-2, the selected set bit-exact on margin-enforced inputs, attention within 2e-2."""
    from conftest import corr_diff, rel_err
    from dsa_multi_layer_indexer_b200 import _lib
    from dsa_multi_layer_indexer_b200.decode import HotPathState, LayerCache

    ctx, heads, topk = 131072, 128, 2048
    g = torch.Generator().manual_seed(0)
    iq = torch.randn(1, 64, 128, generator=g)
    ik = torch.randn(ctx, 128, generator=g)
    w = torch.randn(1, 64, generator=g) / 8
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(iq, ik, w)
    ref_logits = O.indexer_logits_fp8(iq8, ik8, wp, sk)
    sk, ref_row = O.enforce_topk_margin(ref_logits[0], sk, topk)
    sk = sk.float()
    q = torch.randn(1, heads, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(ctx, 576, generator=g).to(torch.bfloat16)
    cache = LayerCache(ik8.view(torch.uint8).view(1, ctx, 128).cuda(), sk.view(1, ctx).cuda(), kv.unsqueeze(0).cuda())
    st = HotPathState(1, heads, 64, ctx, topk, "cuda")
    st.index_q.copy_(iq8.view(torch.uint8).view(1, 64, 128))
    st.index_w.copy_(wp.view(1, 64))
    st.q.copy_(q)
    sm = 192 ** -0.5
    out = st.run(cache, sm).float().cpu()
    torch.cuda.synchronize()
    _lib.check_device_status()
    logits = st.logits[:, :ctx].cpu()
    assert rel_err(logits, ref_row.float().unsqueeze(0)) < 1e-2
    ref_idx = O.select_topk(ref_row.float().unsqueeze(0), topk, pad_value=-1)
    assert torch.equal(st.indices.cpu().long(), ref_idx)
    ref_out = O.sparse_mla_decode(q, kv, ref_idx, [ctx], sm)
    assert rel_err(out, ref_out) < 2e-2
    assert corr_diff(out, ref_out) < 1e-3
    assert int(st.hist.abs().sum()) == 0  # the histogram is re-armed for the next step
