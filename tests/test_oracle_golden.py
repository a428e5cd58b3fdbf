"""Pins the CPU oracle against outputs of the reference's own functions
(tests/golden/*.npz, produced by tests/golden/make_golden.py)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_golden
from oracle import dsa_oracle as O


def test_e4m3_table_matches_torch_cast():
    g = load_golden("fp8_formats.npz")
    ours = O.e4m3_table()
    ref = g["e4m3_table"]
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(ours[ok], ref[ok])


def test_rowwise_quantiser_bit_exact():
    g = load_golden("fp8_formats.npz")
    q, s = O.quantize_e4m3_rowwise(torch.from_numpy(g["x"]))
    assert np.array_equal(q.numpy(), g["xq"])
    assert np.array_equal(s.numpy(), g["xs"])


def test_indexer_fp8_operands_and_logits():
    g = load_golden("indexer_fp8.npz")
    iq8, ik8, wp, sk = O.make_fp8_indexer_inputs(
        torch.from_numpy(g["iq"]), torch.from_numpy(g["ik"]), torch.from_numpy(g["w"]))
    assert np.array_equal(iq8.numpy(), g["iq8"])
    assert np.array_equal(ik8.numpy(), g["ik8"])
    assert np.array_equal(wp.numpy(), g["wp"])
    assert np.array_equal(sk.numpy(), g["sk"])
    logits = O.indexer_logits_fp8(iq8, ik8, wp, sk, chunk=256)
    assert torch.allclose(logits, torch.from_numpy(g["logits"]), rtol=1e-5, atol=1e-5)


def test_sparse_mla_decode():
    g = load_golden("sparse_mla.npz")
    q = bf16_from_bits(g["q"])[0]            # [S,H,576]
    kv = bf16_from_bits(g["kv"])[0, :, 0]    # [N,576]
    idx = torch.from_numpy(g["indices"])
    S, N = q.shape[0], kv.shape[0]
    lens = [(N - S) + s + 1 for s in range(S)]
    out = O.sparse_mla_decode(q, kv, idx, lens, float(g["sm_scale"]))
    assert torch.allclose(out, torch.from_numpy(g["out"])[0], rtol=1e-5, atol=1e-6)


def test_fp32_core_ops():
    g = load_golden("attention_core_f32.npz")
    q, k, w = (torch.from_numpy(g[n]) for n in ("q", "k", "w"))
    logits = O.indexer_logits_f32(q, k, w)
    assert torch.allclose(logits, torch.from_numpy(g["logits"]), rtol=1e-5, atol=1e-5)
    B, S, N = logits.shape
    ref_idx = g["idx"]
    mq, mkv = torch.from_numpy(g["mq"]), torch.from_numpy(g["mkv"])
    for b in range(B):
        lens = list(range(1, S + 1))
        masked = O.mask_beyond(logits[b], lens)
        assert np.array_equal(np.isinf(masked.numpy()), np.isinf(g["masked"][b]))
        ours = O.select_topk(masked, 4, pad_value=N)
        for s in range(S):
            assert sorted(ours[s].tolist()) == sorted(ref_idx[b, s].tolist())
        sm = mq.shape[-1] ** -0.5
        sp = O.sparse_mla_decode(mq[b], mkv[b], torch.from_numpy(ref_idx[b]), lens, sm, value_dim=64)
        assert torch.allclose(sp, torch.from_numpy(g["sparse"])[b], rtol=1e-5, atol=1e-6)
        de = O.dense_mla_decode(mq[b], mkv[b], lens, sm, value_dim=64)
        assert torch.allclose(de, torch.from_numpy(g["dense"])[b], rtol=1e-5, atol=1e-6)


def test_topk_ties_go_to_lower_position():
    logits = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.5, 3.0, float("-inf")]])
    assert O.select_topk(logits, 3, pad_value=-1).tolist() == [[1, 2, 3]]
    assert O.select_topk(logits, 7, pad_value=-1).tolist() == [[0, 1, 2, 3, 4, 5, -1]]


def test_splitk_merge_equals_single_pass():
    torch.manual_seed(0)
    H, V, n, S = 4, 8, 96, 3
    s = torch.randn(H, n) * 3
    v = torch.randn(n, V)
    full = torch.softmax(s, -1) @ v
    acc, m, l = [], [], []
    for c in torch.chunk(torch.arange(n), S):
        sc = s[:, c] * 1.4426950408889634
        mm = sc.max(-1).values
        p = torch.exp2(sc - mm[:, None])
        acc.append(p @ v[c]); m.append(mm); l.append(p.sum(-1))
    # one empty split must be skipped
    acc.append(torch.zeros(H, V)); m.append(torch.full((H,), float("-inf"))); l.append(torch.zeros(H))
    got = O.splitk_merge(torch.stack(acc), torch.stack(m), torch.stack(l))
    assert torch.allclose(got, full, rtol=1e-5, atol=1e-6)


def test_fp8_latent_round_trip():
    torch.manual_seed(0)
    kv = torch.randn(33, 576)
    rows = O.pack_fp8_latent(kv)
    assert rows.shape == (33, 656) and rows.dtype == torch.uint8
    back = O.unpack_fp8_latent(rows).float()
    assert torch.equal(back[:, 512:], kv[:, 512:].to(torch.bfloat16).float())
    assert float((back[:, :512] - kv[:, :512]).abs().max()) < 0.25  # e4m3 step at |x| < 4.5 after scaling


def test_margin_enforcement():
    torch.manual_seed(0)
    logits = torch.randn(4096)
    scale = torch.rand(4096) + 0.5
    s2, l2 = O.enforce_topk_margin(logits, scale, 512, band=2e-2)
    srt = torch.sort(l2, descending=True).values
    gap = float(srt[511] - srt[512])
    assert gap >= 2 * 2e-2 * float(l2.abs().max()) * 0.99
    assert torch.allclose(l2, logits * (s2 / scale), rtol=1e-5, atol=1e-6)


def test_schedule_plan():
    plan = O.schedule_plan([True] * 4, "lagged_fused", "dense")
    assert [p["attend"] for p in plan] == ["dense", "prev", "prev", "prev"]
    assert [p["produce"] for p in plan] == [True, True, True, False]
    plan = O.schedule_plan([False, False, True, True], "lagged_reference", "eager")
    assert [p["attend"] for p in plan] == ["dense", "dense", "prev", "prev"]
    assert [p["produce"] for p in plan] == [False, True, True, False]
    plan = O.schedule_plan([True, True], "baseline", "dense")
    assert all(p["attend"] == "own" and p["produce"] for p in plan)


def test_schedule_plan_depth_follows_the_overlay_narrative():
    """The worked example in the overlay's docstring (patch :3017-3100): with depth k
    the first refresh layer bootstraps, R_1..R_k attend the incoming carry while the
    FIFO fills, and from then on R_n attends the set of R_(n-k)."""
    plan = O.schedule_plan_depth([True] * 7, [True] * 7, "eager", 2)
    assert [p["attend"] for p in plan] == [("layer", 0), ("layer", 0), ("layer", 0), ("layer", 1), ("layer", 2),
                                           ("layer", 3), ("layer", 4)]
    assert all(p["produce"] for p in plan)
    # IndexCache 1/3 retention: skip layers copy the carry, which is the ATTENDED set
    runs = [c == "F" for c in "FSSFSSFSSFSS"]
    plan = O.schedule_plan_depth([True] * 12, runs, "eager", 2)
    att = [p["attend"] for p in plan]
    assert att[:9] == [("layer", 0)] * 9           # R_0 boots; R_1 (layer 3) and R_2 (layer 6) fill
    assert att[9:] == [("layer", 3)] * 3           # R_3 (layer 9) pops R_1's set
    assert [p["produce"] for p in plan] == runs
    # dense cold start queues the first layer's set; dense layers stay dense
    plan = O.schedule_plan_depth([False, True, True, True, True], [True] * 5, "dense", 2)
    assert [p["attend"] for p in plan] == ["dense", "dense", "dense", ("layer", 1), ("layer", 2)]


def _stage_chain(g, inter: bool):
    """The oracle's staging chain up to the rotated bf16 operands."""
    q_raw, k_raw = bf16_from_bits(g["q_raw"]), bf16_from_bits(g["k_raw"])
    cos, sin = torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"])
    q = torch.cat([O.rotary_embed(q_raw[..., :64], cos[:, None, :], sin[:, None, :], inter), q_raw[..., 64:]], dim=-1)
    k = O.layer_norm_128(k_raw, torch.from_numpy(g["norm_w"]), torch.from_numpy(g["norm_b"]), float(g["eps"]))
    k = torch.cat([O.rotary_embed(k[..., :64], cos, sin, inter), k[..., 64:]], dim=-1)
    return O.hadamard_rotate(q), O.hadamard_rotate(k)


def test_indexer_staging_chain_matches_reference_bitwise():
    """LayerNorm -> rotary -> Hadamard rotation, both rotary layouts, against the
    reference's own functions chained in stage_fp8_operands' order."""
    g = load_golden("indexer_stage.npz")
    for inter in (False, True):
        q, k = _stage_chain(g, inter)
        assert torch.equal(q.view(torch.int16), bf16_from_bits(g[f"q_rot_{int(inter)}"]).view(torch.int16))
        assert torch.equal(k.view(torch.int16), bf16_from_bits(g[f"k_rot_{int(inter)}"]).view(torch.int16))


def test_act_quant_definition():
    """Known answers of the block quantiser (inference/modeling/kernels.py:19-117)."""
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    x[0, 5] = 448.0          # amax 448 -> scale 1 (up to the rounding of 1/448)
    x[1, 7] = -3.0           # amax 3
    x[3, :] = 1.0            # row 2 stays all zero: amax clamps at 1e-4
    y, s = O.act_quant_128(x, round_scale=False)
    inv = torch.tensor(1.0 / 448.0, dtype=torch.float32)
    assert torch.equal(s[:, 0], torch.tensor([448.0, 3.0, 1e-4, 1.0]) * inv)
    assert y[0, 5] == 0x7E and y[1, 7] == 0xFE and y[2].eq(0).all() and y[3].eq(0x7E).all()
    y2, s2 = O.act_quant_128(x, round_scale=True)
    # power-of-two scales at or above amax / 448
    assert torch.equal(torch.log2(s2).round(), torch.log2(s2)) and (s2 >= s).all() and (s2 < 2 * s).all()
    assert s2[1, 0] == 2.0 ** -7 and s2[3, 0] == 2.0 ** -8
    deq = O.e4m3_to_f32(y2) * s2
    assert torch.allclose(deq, x.float(), rtol=2 ** -4, atol=0)


def test_indexer_stage_fp8_folds_the_query_scale():
    g = load_golden("indexer_stage.npz")
    q_raw, k_raw = bf16_from_bits(g["q_raw"]), bf16_from_bits(g["k_raw"])
    B, H, _ = q_raw.shape
    torch.manual_seed(3)
    w_raw = torch.randn(B, H)
    cos, sin = torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"])
    for inter in (False, True):
        q8, w, k8, ks = O.indexer_stage_fp8(q_raw, k_raw, w_raw, torch.from_numpy(g["norm_w"]),
                                            torch.from_numpy(g["norm_b"]), float(g["eps"]), cos, sin,
                                            range(B), inter, False, 128 ** -0.5)
        q_rot = bf16_from_bits(g[f"q_rot_{int(inter)}"]).float()
        k_rot = bf16_from_bits(g[f"k_rot_{int(inter)}"]).float()
        q_scale = w / (w_raw * H ** -0.5 * 128 ** -0.5)
        # e4m3: 3 mantissa bits (half a step = 2^-4 relative), subnormal step 2^-9 of the scale
        for deq, ref, sc in ((O.e4m3_to_f32(q8) * q_scale.unsqueeze(-1), q_rot, q_scale.unsqueeze(-1)),
                             (O.e4m3_to_f32(k8) * ks.unsqueeze(-1), k_rot, ks.unsqueeze(-1))):
            assert ((deq - ref).abs() <= ref.abs() * 2 ** -4 + sc.abs() * 2 ** -10 * 1.001).all()


def test_latent_append_matches_reference_and_packing():
    """RMSNorm + rotary of the new latent row against the reference's own modules; the
    packed and fake-quantised forms against each other and pack_fp8_latent."""
    g = load_golden("latent_append.npz")
    kv_a = bf16_from_bits(g["kv_a"])
    B = kv_a.shape[0]
    args = (kv_a, torch.from_numpy(g["norm_w"]), float(g["eps"]), torch.from_numpy(g["cos"]),
            torch.from_numpy(g["sin"]), range(B), True)
    row = O.latent_append_rows(*args, "bf16", False)
    assert torch.equal(row[:, :512].view(torch.int16), bf16_from_bits(g["kv_norm"]).view(torch.int16))
    assert torch.equal(row[:, 512:].view(torch.int16), bf16_from_bits(g["k_pe"]).view(torch.int16))
    packed = O.latent_append_rows(*args, "fp8", False)
    # pack_fp8_latent divides by 448 where act_quant multiplies by 1/448: scales agree to an ulp
    other = O.pack_fp8_latent(row)
    assert packed.shape == (B, 656) and torch.equal(packed[:, 528:], other[:, 528:])
    s_a, s_b = packed[:, 512:528].contiguous().view(torch.float32), other[:, 512:528].contiguous().view(torch.float32)
    assert torch.allclose(s_a, s_b, rtol=2 ** -22, atol=0)
    assert (packed[:, :512] == other[:, :512]).float().mean() > 0.99
    fake = O.latent_append_rows(*args, "bf16_quant", False)
    assert torch.equal(fake.view(torch.int16), O.unpack_fp8_latent(packed).view(torch.int16))
    p2 = O.latent_append_rows(*args, "fp8", True)
    sc = p2[:, 512:528].contiguous().view(torch.float32)
    assert torch.equal(torch.log2(sc).round(), torch.log2(sc))


def test_oracle_at_the_cpu_runnable_configuration():
    """The oracle's fp32 decode path at the reference's own CPU-runnable size (context 4096,
    64 x 128 indexer, top-2048, 16 heads x 576, scale 1/sqrt(192)) against what the reference's
    indexer_logits / select_topk / _attend produced from the same seeded inputs."""
    g = load_golden("config1_decode.npz")
    torch.manual_seed(0)
    n = 4096
    iq = torch.randn(1, 1, 64, 128)
    ik = torch.randn(1, n, 128)
    w = torch.randn(1, 1, 64) / 8
    q = torch.randn(1, 1, 16, 576)
    kv = torch.randn(1, n, 576)
    sums = [float(t.double().sum()) for t in (iq, ik, w, q, kv)]
    assert sums == pytest.approx(g["sums"].tolist(), rel=1e-12)
    ik = ik * torch.from_numpy(g["key_scale"]).view(1, -1, 1)
    logits = O.indexer_logits_f32(iq, ik, w)[0]
    assert torch.allclose(logits[0], torch.from_numpy(g["logits"]), rtol=1e-5, atol=1e-5)
    idx = O.select_topk(logits, 2048, pad_value=-1)
    assert torch.equal(idx[0].int(), torch.from_numpy(g["idx"]))
    out = O.sparse_mla_decode(q[0], kv[0], idx, [n], 192 ** -0.5)
    assert torch.allclose(out[0], torch.from_numpy(g["out"]), rtol=1e-4, atol=1e-5)
