"""GPU parity tests of the tcgen05 sparse MLA decode kernel (64-head CTAs, S and
O^T in tensor memory) against the CPU oracle and against the mma.sync kernel on
the same inputs. DSA_MLA_TC=2 forces the tcgen05 kernel for every head count
that is a multiple of 64, =0 keeps the mma.sync kernel, =1 (default) picks by
problem size. Tolerance: attention output <= 2e-2 relative (bf16)."""

from __future__ import annotations

import pytest
import torch

from conftest import corr_diff, rel_err
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-2


@pytest.fixture(scope="module")
def ops():
    from dsa_multi_layer_indexer_b200 import _lib, ops as _ops

    _lib.lib()  # fail loudly if the library is missing
    yield _ops
    _lib.check_device_status()


def dev(t: torch.Tensor) -> torch.Tensor:
    return t.cuda().contiguous()


def decode(ops, monkeypatch, mode, *args, **kw):
    monkeypatch.setenv("DSA_MLA_TC", mode)
    out = ops.sparse_mla_decode(*args, **kw).float().cpu()
    from dsa_multi_layer_indexer_b200 import _lib
    _lib.check_device_status()
    return out


@pytest.mark.parametrize("H,topk,n,nsplit", [(64, 64, 300, 1), (64, 128, 4096, 1), (64, 200, 1000, 3),
                                             (128, 2048, 8192, 8), (128, 2048, 3000, 5), (64, 80, 100, 2),
                                             (192, 512, 2000, 4)])
def test_tc_matches_oracle_and_mma_sync(ops, monkeypatch, H, topk, n, nsplit):
    torch.manual_seed(H + topk + nsplit)
    q = torch.randn(1, H, 576).to(torch.bfloat16)
    kv = torch.randn(n, 576).to(torch.bfloat16)
    idx = torch.full((1, topk), -1, dtype=torch.int32)
    take = min(topk, n)
    idx[0, :take] = torch.randperm(n)[:take].int()
    idx[0, ::17] = n + 5  # entries beyond the sequence are skipped
    idx[0, 3::29] = -1    # and so is padding
    sm = 192 ** -0.5
    tc = decode(ops, monkeypatch, "2", dev(q), dev(kv), dev(idx), sm, nsplit=nsplit)
    legacy = decode(ops, monkeypatch, "0", dev(q), dev(kv), dev(idx), sm, nsplit=nsplit)
    ref = O.sparse_mla_decode(q, kv, idx, [n], sm)
    assert rel_err(tc, ref) < ATTN_TOL
    assert corr_diff(tc, ref) < 1e-3
    assert rel_err(tc, legacy) < ATTN_TOL


def test_tc_ragged_batch_and_empty_rows(ops, monkeypatch):
    torch.manual_seed(21)
    B, H, n, topk = 5, 64, 2500, 1024
    q = torch.randn(B, H, 576).to(torch.bfloat16)
    kv = torch.randn(B, n, 576).to(torch.bfloat16)
    lens = [2500, 1, 1300, 0, 64]
    idx = torch.stack([torch.randperm(n)[:topk] for _ in range(B)]).int()
    idx[4] = -1  # a row whose selection is all padding
    seq = dev(torch.tensor(lens, dtype=torch.int32))
    sm = 576 ** -0.5
    both = decode(ops, monkeypatch, "2", dev(q), dev(kv), dev(idx), sm, seq, nsplit=4)
    assert torch.isfinite(both).all()
    assert float(both[3].abs().max()) == 0.0 and float(both[4].abs().max()) == 0.0
    for b in range(B):
        one = decode(ops, monkeypatch, "2", dev(q[b:b + 1]), dev(kv[b:b + 1]), dev(idx[b:b + 1]), sm, seq[b:b + 1],
                     nsplit=4)
        assert torch.equal(one[0], both[b])  # a row does not depend on its batch
        if lens[b] > 0 and b != 4:
            ref = O.sparse_mla_decode(q[b:b + 1], kv[b], idx[b:b + 1], [lens[b]], sm)
            assert rel_err(both[b:b + 1], ref) < ATTN_TOL


def test_tc_dense_mode(ops, monkeypatch):
    torch.manual_seed(22)
    H, n = 64, 700
    q = torch.randn(1, H, 576).to(torch.bfloat16)
    kv = torch.randn(n, 576).to(torch.bfloat16)
    seq = dev(torch.tensor([650], dtype=torch.int32))
    got = decode(ops, monkeypatch, "2", dev(q), dev(kv), None, 0.07, seq, nsplit=3)
    ref = O.dense_mla_decode(q, kv, [650], 0.07)
    assert rel_err(got, ref) < ATTN_TOL


def test_tc_fp8_latent_rows(ops, monkeypatch):
    torch.manual_seed(23)
    H, n, topk = 128, 3000, 2048
    q = torch.randn(2, H, 576).to(torch.bfloat16)
    rows = O.pack_fp8_latent(torch.randn(n, 576))
    idx = torch.stack([torch.randperm(n)[:topk] for _ in range(2)]).int()
    idx[:, ::13] = -1
    sm = 192 ** -0.5
    seq = dev(torch.tensor([n, n - 700], dtype=torch.int32))
    kv = dev(rows).unsqueeze(0).expand(2, -1, -1).contiguous()
    got = decode(ops, monkeypatch, "2", dev(q), kv, dev(idx), sm, seq, nsplit=4)
    legacy = decode(ops, monkeypatch, "0", dev(q), kv, dev(idx), sm, seq, nsplit=4)
    for b, ln in enumerate((n, n - 700)):
        ref = O.sparse_mla_decode(q[b:b + 1], O.unpack_fp8_latent(rows), idx[b:b + 1], [ln], sm)
        assert rel_err(got[b:b + 1], ref) < ATTN_TOL
        assert corr_diff(got[b:b + 1], ref) < 1e-3
    assert rel_err(got, legacy) < ATTN_TOL


@pytest.mark.parametrize("mult", [20.0, 80.0])
def test_tc_runaway_maximum_rescales(ops, monkeypatch, mult):
    """Keys late in the list have logits far above the first tile's maximum, which
    the kernel keeps as its softmax reference: the rescale of O^T must kick in."""
    torch.manual_seed(24)
    H, n, topk = 64, 4096, 1024
    q = torch.randn(2, H, 576).to(torch.bfloat16)
    kvf = torch.randn(2, n, 576)
    kvf[:, n // 2:] *= mult
    kv = kvf.to(torch.bfloat16)
    idx = torch.stack([torch.sort(torch.randperm(n)[:topk]).values for _ in range(2)]).int()
    got = decode(ops, monkeypatch, "2", dev(q), dev(kv), dev(idx), 0.07, nsplit=1)
    for b in range(2):
        ref = O.sparse_mla_decode(q[b:b + 1], kv[b], idx[b:b + 1], [n], 0.07)
        assert torch.isfinite(got[b]).all()
        assert rel_err(got[b:b + 1], ref) < ATTN_TOL


def test_size_based_dispatch_matches(ops, monkeypatch):
    """Default mode: eight rows of 128 heads x 2048 keys cross the tile threshold and
    run on the tcgen05 kernel; the result agrees with the mma.sync kernel."""
    torch.manual_seed(25)
    B, H, n, topk = 8, 128, 6000, 2048
    q = torch.randn(B, H, 576).to(torch.bfloat16)
    kv = torch.randn(B, n, 576).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(n)[:topk] for _ in range(B)]).int()
    sm = 192 ** -0.5
    auto = decode(ops, monkeypatch, "1", dev(q), dev(kv), dev(idx), sm)
    legacy = decode(ops, monkeypatch, "0", dev(q), dev(kv), dev(idx), sm)
    forced = decode(ops, monkeypatch, "2", dev(q), dev(kv), dev(idx), sm)
    assert rel_err(auto, legacy) < ATTN_TOL
    assert torch.equal(auto, forced)
