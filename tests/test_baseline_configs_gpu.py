"""The benchmark configurations at their own sizes, through the C ABI, against the
CPU oracle and the reference-generated fixtures.

* configuration 1: the reference's CPU-runnable single-layer decode, fp32, context 4096,
  64 indexer heads x 128, top-2048, 16 MLA heads x 576 -> [16, 512]
  (``dsa_indexer_scan_f32`` -> ``dsa_topk_select`` -> ``dsa_sparse_mla_f32``) against
  ``tests/golden/config1_decode.npz``, which the reference's own ``indexer_logits`` /
  ``select_topk`` / ``_attend`` produced (src/lagged_indexer_dsa/attention_core.py:27-118);
* configuration 5: a 262144-key context whose scan is split over 2 / 4 / 8 KV ranges, each
  range's local top-2048 merged to the global one (the ranks emulated as slices on one GPU),
  and the 1-of-4 retention plan over an 8-layer stack.

(Configuration 2 at full size lives in test_decode_gpu.py, configuration 4 in
test_serving_gpu.py, configuration 3's dimensions in test_model_gpu.py.)
"""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, rel_err
from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from dsa_multi_layer_indexer_b200 import ops as _ops
    return _ops


def config1_inputs():
    torch.manual_seed(0)
    n = 4096
    iq = torch.randn(1, 1, 64, 128)
    ik = torch.randn(1, n, 128)
    w = torch.randn(1, 1, 64) / 8
    q = torch.randn(1, 1, 16, 576)
    kv = torch.randn(1, n, 576)
    return iq, ik, w, q, kv


def test_config1_fp32_decode_at_its_exact_shape(ops):
    g = load_golden("config1_decode.npz")
    iq, ik, w, q, kv = config1_inputs()
    sums = [float(t.double().sum()) for t in (iq, ik, w, q, kv)]
    assert sums == pytest.approx(g["sums"].tolist(), rel=1e-12), "the seeded inputs differ from the fixture's"
    ik = ik * torch.from_numpy(g["key_scale"]).view(1, -1, 1)  # the margin-enforced keys
    dev = "cuda"
    logits = ops.indexer_scan_f32(iq[0].to(dev), w[0].to(dev), ik.to(dev))
    idx = ops.topk_select(logits, 2048)
    out = ops.sparse_mla_f32(q[0].to(dev), kv.to(dev), idx, 512, 192 ** -0.5)
    torch.cuda.synchronize()
    ref_logits = torch.from_numpy(g["logits"])
    assert rel_err(logits.cpu()[0], ref_logits) < 1e-5
    assert torch.equal(idx.cpu()[0], torch.from_numpy(g["idx"]))  # ascending positions == the sorted reference set
    assert rel_err(out.cpu()[0], torch.from_numpy(g["out"])) < 2e-4
    # and the oracle agrees with the reference on the same inputs
    o_logits = O.indexer_logits_f32(iq, ik, w)[0]
    o_idx = O.select_topk(o_logits, 2048, pad_value=-1)
    assert torch.equal(o_idx[0].int(), torch.from_numpy(g["idx"]))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_config5_sequence_sharded_selection_at_262144_keys(ops, world):
    """Context 262144, FP8 keys with a margin around the rank-2048 cutoff: every shard's local
    top-2048 as (global position, logit), concatenated in rank order and merged through the
    index map, is the oracle's global selection bit for bit, and equals the unsharded launch."""
    from dsa_multi_layer_indexer_b200.parallel import key_range

    n, topk = 262144, 2048
    torch.manual_seed(5)
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(torch.randn(1, 64, 128), torch.randn(n, 128),
                                                 torch.randn(1, 64) / 8)
    ref_logits = O.indexer_logits_fp8(iq8, ik8, wp, sk, chunk=32768)
    sk, ref_row = O.enforce_topk_margin(ref_logits[0], sk, topk)
    want = O.select_topk(ref_row.unsqueeze(0), topk, pad_value=-1)
    iq8, ik8, wp, sk = (t.cuda() for t in (iq8, ik8, wp, sk))
    full_logits = ops.indexer_scan_fp8(iq8, wp, ik8, sk)
    assert rel_err(full_logits.cpu(), ref_row.unsqueeze(0)) < 1e-2
    full = ops.topk_select(full_logits, topk)
    assert torch.equal(full.cpu().long(), want)
    ci, cv = [], []
    for r in range(world):
        lo, hi = key_range(r, world, n)
        assert (lo, hi) == (r * n // world, (r + 1) * n // world)
        hist = torch.zeros(1, ops.HIST_BINS, dtype=torch.int32, device="cuda")
        logits = ops.indexer_scan_fp8(iq8, wp, ik8[lo:hi].contiguous(), sk[lo:hi].contiguous(), hist=hist)
        i, v = ops.topk_select(logits, topk, hist=hist, index_offset=lo, return_values=True)
        ci.append(i)
        cv.append(v)
    merged = ops.topk_select(torch.cat(cv, 1).contiguous(), topk, index_map=torch.cat(ci, 1).contiguous())
    torch.cuda.synchronize()
    assert torch.equal(merged.cpu().long(), want)
    from dsa_multi_layer_indexer_b200 import _lib
    _lib.check_device_status()


def test_config5_one_in_four_retention_over_eight_layers():
    """Indexers on every 4th layer of an 8-layer stack: layers 0 and 4 produce a selection,
    the six others reuse the carried one, under the serial and the lagged schedule."""
    import dataclasses

    import dsa_multi_layer_indexer_b200 as D
    from dsa_multi_layer_indexer_b200.model import parse_retention

    assert parse_retention("4", 8) == [True, False, False, False, True, False, False, False]
    cfg = dataclasses.replace(D.SMALL_CONFIG, num_hidden_layers=8)
    torch.manual_seed(3)
    model = D.DSAModel(cfg).eval().cuda()
    B, S0 = 2, 40
    st = model.init_decode(B, 48, fp8=False, retention="4")
    model.prefill(st, torch.randn(B, S0, cfg.hidden_size, device="cuda"))
    for mode, cold in ((D.ScheduleMode.BASELINE, D.ColdStartPolicy.DENSE),
                       (D.ScheduleMode.LAGGED_FUSED, D.ColdStartPolicy.EAGER)):
        rec = {}
        model.decode_step(st, torch.randn(B, cfg.hidden_size, device="cuda"), mode, cold, record=rec)
        used, made = rec["used"], rec["produced"]
        assert [m is not None for m in made] == [True, False, False, False, True, False, False, False]
        if mode is D.ScheduleMode.BASELINE:
            for l in (1, 2, 3):
                assert torch.equal(used[l], made[0])
            for l in (5, 6, 7):
                assert torch.equal(used[l], made[4])
        else:  # lagged: a layer attends what the latest indexer layer BEFORE it produced
            for l in (1, 2, 3, 4):
                assert torch.equal(used[l], made[0])
            for l in (5, 6, 7):
                assert torch.equal(used[l], made[4])
