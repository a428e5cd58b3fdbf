"""Multi-GPU logic: shard arithmetic and the candidate exchange on CPU (gloo,
world size 2), the sequence-sharded selection emulated on one GPU, and the real
NCCL path when two GPUs are present."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dsa_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ranges_cover_everything():
    from dsa_multi_layer_indexer_b200.parallel import head_range, key_range

    for world in (1, 2, 4, 8):
        assert [head_range(r, world, 128) for r in range(world)][-1][1] == 128
        for n in (1, 127, 128, 1000, 131072, 262144, 200001):
            spans = [key_range(r, world, n) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(lo % 128 == 0 for lo, hi in spans if hi > lo)
    with pytest.raises(ValueError):
        head_range(0, 3, 128)


def _gloo_worker(rank: int, world: int, port: int, n: int, topk: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dsa_multi_layer_indexer_b200.parallel import interleave_gathered, key_range

        g = torch.Generator().manual_seed(0)  # every rank draws the same global logits
        logits = torch.randn(2, n, generator=g)
        logits[1, ::3] = logits[1, 0]  # heavy ties across shards
        lo, hi = key_range(rank, world, n)
        # local top-k as (global position, value) in ascending position order, padded
        local = O.select_topk(logits[:, lo:hi], topk, pad_value=-1)
        cand_idx = torch.where(local >= 0, local + lo, local).to(torch.int32)
        cand_val = torch.full((2, topk), float("-inf"))
        for r in range(2):
            keep = local[r] >= 0
            cand_val[r, keep] = logits[r, lo:hi][local[r, keep]]
        gi = torch.empty(world, 2, topk, dtype=torch.int32)
        gv = torch.empty(world, 2, topk)
        dist.all_gather_into_tensor(gi.view(-1), cand_idx.view(-1))
        dist.all_gather_into_tensor(gv.view(-1), cand_val.view(-1))
        idxs = interleave_gathered(gi, world, 2, topk)
        vals = interleave_gathered(gv, world, 2, topk)
        # merge = top-k of the candidates, ties to the lower slot (= lower position)
        pick = O.select_topk(vals, topk, pad_value=-1)
        merged = torch.gather(idxs.long(), 1, pick.clamp(min=0))
        want = O.select_topk(logits, topk, pad_value=-1)
        for r in range(2):
            assert sorted(merged[r].tolist()) == want[r].tolist(), f"rank {rank} row {r}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,topk", [(4096, 256), (1000, 64)])
def test_candidate_exchange_gloo_world2(n, topk):
    mp.spawn(_gloo_worker, args=(2, _free_port(), n, topk), nprocs=2, join=True)


@pytest.mark.gpu
def test_sequence_sharded_selection_emulated_on_one_gpu():
    """Four 'ranks' as slices of one cache: local top-k with a position offset,
    concatenation in rank order, merge through index_map == global selection."""
    from dsa_multi_layer_indexer_b200 import ops
    from dsa_multi_layer_indexer_b200.parallel import key_range

    n, topk, world = 40000, 2048, 4
    torch.manual_seed(0)
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(torch.randn(1, 64, 128), torch.randn(n, 128),
                                                 torch.randn(1, 64) / 8)
    iq8, ik8, wp, sk = (t.cuda() for t in (iq8, ik8, wp, sk))
    full = ops.topk_select(ops.indexer_scan_fp8(iq8, wp, ik8, sk), topk)
    ci, cv = [], []
    for r in range(world):
        lo, hi = key_range(r, world, n)
        logits = ops.indexer_scan_fp8(iq8, wp, ik8[lo:hi].contiguous(), sk[lo:hi].contiguous())
        i, v = ops.topk_select(logits, topk, index_offset=lo, return_values=True)
        ci.append(i)
        cv.append(v)
    merged = ops.topk_select(torch.cat(cv, 1).contiguous(), topk, index_map=torch.cat(ci, 1).contiguous())
    assert torch.equal(merged, full)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_store_exchange_emulated_on_one_gpu(world):
    """The exchange kernels with every "rank" on one GPU: each rank's local top-k stores its
    candidates into all ranks' gather buffers and posts its flags, then each rank's merge finds
    the flags already there and selects. Three steps with different logits (the two buffer
    parities, then the first one again), ragged rows, one empty shard: every rank ends with the
    oracle's global selection. The ranks' launches are enqueued one after the other on one
    stream, every push before the first merge, so no kernel ever waits for a later one."""
    from dsa_multi_layer_indexer_b200 import _lib, ops
    from dsa_multi_layer_indexer_b200.parallel import key_range

    rows, topk, n = 3, 512, 20000
    xs = ops.CandidateExchange.local_group(rows, topk, world, "cuda")
    outs = [torch.full((rows, topk), -7, dtype=torch.int32, device="cuda") for _ in range(world)]
    lens = [n, n // 2 + 17, 300]  # row 2: only the first shard sees any key
    for step in range(3):
        g = torch.Generator().manual_seed(100 + step)
        logits = torch.randn(rows, n, generator=g)
        logits[1, ::5] = logits[1, 0]  # ties across shards
        want = O.select_topk(O.mask_beyond(logits, lens), topk, pad_value=-1)
        dl = logits.cuda()
        for r in range(world):
            lo, hi = key_range(r, world, n)
            local = dl[:, lo:hi].contiguous()
            local_lens = torch.tensor([max(0, min(l, hi) - lo) for l in lens], dtype=torch.int32, device="cuda")
            xs[r].push(local, local_lens, index_offset=lo)
        for r in range(world):
            xs[r].merge(outs[r])
        torch.cuda.synchronize()
        _lib.check_device_status()
        for r in range(world):
            assert torch.equal(outs[r].cpu().long(), want), f"step {step} rank {r}"
        assert xs[0].sent.tolist() == [step + 1] * rows and xs[0].seen.tolist() == [step + 1] * rows


@pytest.mark.gpu
def test_merge_wait_runs_out_when_a_rank_never_posts():
    """Failure detection without a fault: rank 1 of a two-rank exchange never pushes. Rank 0's merge
    waits for that flag with a limit of two milliseconds, gives up, sets the status word and returns;
    the host call that reads the status raises, and the context stays usable."""
    from dsa_multi_layer_indexer_b200 import _lib, ops

    rows, topk = 2, 64
    xs = ops.CandidateExchange.local_group(rows, topk, 2, "cuda", wait_limit_s=0.002)
    out = torch.full((rows, topk), -7, dtype=torch.int32, device="cuda")
    xs[0].push(torch.randn(rows, 1000, device="cuda"))
    _lib.check_device_status()
    xs[0].merge(out)  # rank 1 posted nothing
    with pytest.raises(_lib.DsaError) as err:
        _lib.check_device_status()
    assert err.value.status == -4
    _lib.check_device_status()  # read and cleared
    # the context is alive: rank 1 catches up, the next step completes in time
    xs[1].push(torch.randn(rows, 1000, device="cuda"))
    xs[1].merge(out)
    xs[0].push(torch.randn(rows, 1000, device="cuda"))
    xs[1].push(torch.randn(rows, 1000, device="cuda"))
    xs[0].merge(out)
    _lib.check_device_status()
    assert int((out >= 0).sum()) == rows * topk


def _nccl_worker(rank: int, world: int, port: int, n: int, topk: int, out_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from dsa_multi_layer_indexer_b200 import ops
        from dsa_multi_layer_indexer_b200.parallel import SeqShardedIndexer, head_range, key_range

        torch.manual_seed(0)
        iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(torch.randn(2, 64, 128), torch.randn(n, 128),
                                                     torch.randn(2, 64) / 8)
        q = torch.randn(2, 32, 576).to(torch.bfloat16)
        kv = torch.randn(n, 576).to(torch.bfloat16)
        iq8, ik8, wp, sk, q, kv = (t.cuda() for t in (iq8, ik8, wp, sk, q, kv))
        lo, hi = key_range(rank, world, n)
        keys = ik8[lo:hi].unsqueeze(0).expand(2, -1, -1).contiguous()
        scales = sk[lo:hi].unsqueeze(0).expand(2, -1).contiguous()
        picked = []
        for exchange in ("p2p", "nccl"):
            idxr = SeqShardedIndexer(2, topk, hi - lo, lo, "cuda", exchange=exchange)
            sel = idxr.select(iq8, wp, keys, scales).clone()
            # the same step captured (one graph with the peer-store exchange, two graphs around the
            # all-gather with NCCL), with a consumer behind the merge
            seen = torch.zeros_like(sel)
            step = idxr.capture(iq8, wp, keys, scales, after=lambda idx: seen.copy_(idx))
            for _ in range(3):
                seen.zero_()
                idxr.indices.fill_(-7)
                sel_g = step().clone()
                torch.cuda.synchronize()
                assert torch.equal(sel_g, sel) and torch.equal(seen, sel), exchange
            picked.append(sel)
            dist.barrier()
        from dsa_multi_layer_indexer_b200 import _lib
        _lib.check_device_status()
        assert torch.equal(picked[0], picked[1])
        sel = picked[0]
        h0, h1 = head_range(rank, world, 32)
        kv2 = kv.unsqueeze(0).expand(2, -1, -1).contiguous()
        part = ops.sparse_mla_decode(q[:, h0:h1].contiguous(), kv2, sel, 0.07, nsplit=8)
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        if rank == 0:
            ik2 = ik8.unsqueeze(0).expand(2, -1, -1).contiguous()
            sk2 = sk.unsqueeze(0).expand(2, -1).contiguous()
            want_sel = ops.topk_select(ops.indexer_scan_fp8(iq8, wp, ik2, sk2), topk)
            want_out = ops.sparse_mla_decode(q, kv2, want_sel, 0.07, nsplit=8)
            ok = torch.equal(sel, want_sel) and torch.equal(torch.cat(gathered, 1), want_out)
            with open(out_path, "w") as f:
                f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_sequence_sharded_indexer_and_tp_heads_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "result.txt"
    mp.spawn(_nccl_worker, args=(2, _free_port(), 30000, 2048, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
