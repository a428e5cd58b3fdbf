"""GPU tests of the layer / model API: the reference's schedules on the SMALL
preset against reference-generated goldens, the decode path against the
full-sequence forward, the two-stream lagged schedule and its CUDA graph."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def D():
    import dsa_multi_layer_indexer_b200 as pkg
    from dsa_multi_layer_indexer_b200 import _lib

    _lib.lib()
    yield pkg
    _lib.check_device_status()


def small_model(D, seed):
    torch.manual_seed(seed)  # same construction order as the reference -> same weights
    return D.DSAModel(D.SMALL_CONFIG).eval().cuda()


def sets_equal(a: torch.Tensor, b: np.ndarray, sentinel: int) -> float:
    """Fraction of (batch, query) rows whose selected sets agree exactly."""
    a = a.cpu().numpy().reshape(-1, a.shape[-1])
    b = b.reshape(-1, b.shape[-1])
    same = 0
    for ra, rb in zip(a, b):
        sa = set(int(v) for v in ra if 0 <= v < sentinel)
        sb = set(int(v) for v in rb if 0 <= v < sentinel)
        same += sa == sb
    return same / len(a)


@pytest.mark.parametrize("seed", [0, 7])
def test_forward_matches_reference_goldens(D, seed):
    g = load_golden("model_small.npz")
    model = small_model(D, seed)
    x = torch.from_numpy(g[f"x_{seed}"]).cuda()
    S = x.shape[1]
    for mode in D.ScheduleMode:
        for cold in D.ColdStartPolicy:
            with torch.no_grad():
                tr = model(x, mode, cold_start=cold, record=True)
            key = f"{seed}_{mode.value}_{cold.value}"
            ref_h = torch.from_numpy(g[f"hidden_{key}"])
            assert rel_err(tr.final_hidden.cpu(), ref_h) < 2e-4, key
            for li, (u, p) in enumerate(zip(tr.indices_used, tr.indices_produced)):
                assert (u is None) == (f"used_{key}_{li}" not in g.files)
                assert (p is None) == (f"produced_{key}_{li}" not in g.files)
                if p is not None:
                    assert p.dtype == torch.int64 and p.shape == (1, S, D.SMALL_CONFIG.index_topk)
                    assert sets_equal(p, g[f"produced_{key}_{li}"], S) == 1.0, (key, li)
                if u is not None:
                    assert sets_equal(u, g[f"used_{key}_{li}"], S) == 1.0, (key, li)


def test_lagged_fused_equals_lagged_reference_and_is_causal(D):
    model = small_model(D, 1)
    torch.manual_seed(5)
    x = torch.randn(2, 24, D.SMALL_CONFIG.hidden_size, device="cuda")
    with torch.no_grad():
        a = model(x, D.ScheduleMode.LAGGED_FUSED, record=True)
        b = model(x, D.ScheduleMode.LAGGED_REFERENCE, record=True)
        base = model(x, D.ScheduleMode.BASELINE)
    assert torch.equal(a.final_hidden, b.final_hidden)
    for ia, ib in zip(a.indices_produced, b.indices_produced):
        assert (ia is None) == (ib is None)
        if ia is not None:
            assert torch.equal(ia, ib)
    assert not torch.allclose(a.final_hidden, base)  # the lag changes the result
    S = x.shape[1]
    pos = torch.arange(S, device="cuda").view(1, S, 1)
    for u in a.indices_used:
        if u is not None:
            real = u < S
            assert bool((u[real] <= pos.expand_as(u)[real]).all())
    assert a.indices_produced[-1] is None  # the last layer has no consumer


@pytest.mark.parametrize("mode_name", ["BASELINE", "LAGGED_FUSED"])
def test_decode_equals_full_forward(D, mode_name):
    mode = D.ScheduleMode[mode_name]
    cold = D.ColdStartPolicy.EAGER
    model = small_model(D, 3)
    torch.manual_seed(8)
    B, S, S0 = 2, 30, 20
    x = torch.randn(B, S, D.SMALL_CONFIG.hidden_size, device="cuda")
    with torch.no_grad():
        full = model(x, mode, cold_start=cold)
    st = model.init_decode(B, 64, fp8=False)
    pre = model.prefill(st, x[:, :S0], mode, cold)
    assert rel_err(pre.cpu(), full[:, :S0].cpu()) < 1e-4
    for t in range(S0, S):
        out = model.decode_step(st, x[:, t], mode, cold)
        assert rel_err(out.cpu(), full[:, t].cpu()) < 2e-4, t
    assert st.positions.tolist() == [S, S]


def test_lagged_overlap_graph_and_eager_agree(D):
    model = small_model(D, 4)
    torch.manual_seed(9)
    B, S0, steps = 3, 16, 6
    hid = D.SMALL_CONFIG.hidden_size
    prompt = torch.randn(B, S0, hid, device="cuda")
    toks = torch.randn(steps, B, hid, device="cuda")
    mode, cold = D.ScheduleMode.LAGGED_FUSED, D.ColdStartPolicy.DENSE

    def run(overlap, graph):
        st = model.init_decode(B, 40, fp8=False)
        model.prefill(st, prompt, mode, cold)
        outs = []
        if graph:
            g, x_in, x_out = model.capture_decode(st, mode, cold, overlap=overlap)
            for t in range(steps):
                x_in.copy_(toks[t])
                g.replay()
                outs.append(x_out.clone())
        else:
            for t in range(steps):
                outs.append(model.decode_step(st, toks[t], mode, cold, overlap=overlap).clone())
        torch.cuda.synchronize()
        assert st.positions.tolist() == [S0 + steps] * B
        return torch.stack(outs)

    serial = run(False, False)
    two_streams = run(True, False)
    graphed = run(True, True)
    assert torch.equal(serial, two_streams)
    assert torch.equal(serial, graphed)


def test_retention_pattern_carries_the_selection(D):
    model = small_model(D, 5)
    torch.manual_seed(10)
    B, S0 = 1, 24
    hid = D.SMALL_CONFIG.hidden_size
    st = model.init_decode(B, 32, fp8=False, retention="FSSFSS")
    model.prefill(st, torch.randn(B, S0, hid, device="cuda"))
    rec = {}
    model.decode_step(st, torch.randn(B, hid, device="cuda"), D.ScheduleMode.BASELINE, record=rec)
    used, made = rec["used"], rec["produced"]
    assert [m is not None for m in made] == [True, False, False, True, False, False]
    assert torch.equal(used[1], made[0]) and torch.equal(used[2], made[0])
    assert torch.equal(used[4], made[3]) and torch.equal(used[5], made[3])
    rec = {}
    model.decode_step(st, torch.randn(B, hid, device="cuda"), D.ScheduleMode.LAGGED_FUSED,
                      D.ColdStartPolicy.EAGER, record=rec)
    used, made = rec["used"], rec["produced"]
    assert [m is not None for m in made] == [True, False, False, True, False, False]
    assert torch.equal(used[1], made[0]) and torch.equal(used[3], made[0])  # the F layer attends the carry
    assert torch.equal(used[4], made[3])


@pytest.mark.parametrize("cold,pattern,depth", [("eager", None, 2), ("dense", None, 2), ("eager", "FSFSFS", 2),
                                                 ("eager", None, 3)])
def test_lag_depth_k_follows_the_plan_and_overlaps(D, cold, pattern, depth):
    """Every layer attends exactly the set the depth-k plan names; one stream, the side
    stream and a captured graph give identical hidden states."""
    from oracle import dsa_oracle as O

    model = small_model(D, 6)
    n_layers = len(model.layers)
    assert n_layers == 6
    is_dsa = [t is D.AttentionType.DSA for t in model.config.resolved_attention_types]
    torch.manual_seed(12)
    B, S0 = 2, 20
    hid = D.SMALL_CONFIG.hidden_size
    prompt = torch.randn(B, S0, hid, device="cuda")
    tok = torch.randn(3, B, hid, device="cuda")
    mode = D.ScheduleMode.LAGGED_FUSED
    policy = D.ColdStartPolicy.EAGER if cold == "eager" else D.ColdStartPolicy.DENSE

    def fresh():
        st = model.init_decode(B, 32, fp8=False, retention=pattern)
        model.prefill(st, prompt)
        return st

    st = fresh()
    rec = {}
    serial = model.decode_step(st, tok[0], mode, policy, overlap=False, record=rec, lag_depth=depth).clone()
    plan = O.schedule_plan_depth(is_dsa, st.runs_indexer, cold, depth)
    for li, p in enumerate(plan):
        assert (rec["produced"][li] is not None) == p["produce"], li
        if p["attend"] == "dense":
            assert rec["used"][li] is None, li
        else:
            assert torch.equal(rec["used"][li], rec["produced"][p["attend"][1]]), li
    st = fresh()
    overlapped = model.decode_step(st, tok[0], mode, policy, overlap=True, lag_depth=depth)
    assert torch.equal(serial, overlapped)
    st = fresh()
    g, x_in, x_out = model.capture_decode(st, mode, policy, overlap=True, lag_depth=depth)
    x_in.copy_(tok[0])
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(serial, x_out)
    with pytest.raises(ValueError):
        model.decode_step(st, tok[1], D.ScheduleMode.BASELINE, lag_depth=2)


def production_config(D, layers=3):
    return D.DSAConfig(hidden_size=256, num_hidden_layers=layers, num_attention_heads=16, q_lora_rank=96,
                       kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32,
                       index_n_heads=16, index_head_dim=128, index_topk=64, intermediate_size=512,
                       first_k_dense_replace=0)


def test_production_geometry_fp8_bf16_path(D):
    """FP8 scan + bf16 split-K attention behind the same model API at reduced width: decode
    follows the fp32 kernels within bf16 tolerance and picks nearly the same keys."""
    cfg = production_config(D)
    torch.manual_seed(11)
    ref_model = D.DSAModel(cfg).eval().cuda()
    fast = D.DSAModel(cfg).eval().cuda().to(torch.bfloat16)
    fast.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref_model.state_dict().items()})
    ref_model.load_state_dict({k: v.float() for k, v in fast.state_dict().items()})  # same rounded weights
    B, S0, steps = 2, 200, 4
    torch.manual_seed(12)
    prompt = torch.randn(B, S0, cfg.hidden_size, device="cuda")
    toks = torch.randn(steps, B, cfg.hidden_size, device="cuda")
    mode, cold = D.ScheduleMode.LAGGED_FUSED, D.ColdStartPolicy.EAGER
    s_ref = ref_model.init_decode(B, 256, fp8=False)
    s_fast = fast.init_decode(B, 256)
    assert s_fast.fp8
    ref_model.prefill(s_ref, prompt, mode, cold)
    fast.prefill(s_fast, prompt.to(torch.bfloat16), mode, cold)
    overlaps = []
    for t in range(steps):
        ra, rb = {}, {}
        a = ref_model.decode_step(s_ref, toks[t], mode, cold, record=ra)
        b = fast.decode_step(s_fast, toks[t].to(torch.bfloat16), mode, cold, record=rb)
        assert rel_err(b.float().cpu(), a.cpu()) < 6e-2
        for ia, ib in zip(ra["produced"], rb["produced"]):
            if ia is not None:
                for r in range(B):
                    sa, sb = set(ia[r].tolist()) - {-1}, set(ib[r].tolist()) - {-1}
                    overlaps.append(len(sa & sb) / max(1, len(sa | sb)))
    assert min(overlaps) > 0.6 and sum(overlaps) / len(overlaps) > 0.8


def test_lagged_chained_on_one_stream_equals_serial(D):
    """The lagged schedule as one chain on one stream (each layer's attention enqueued behind the
    layer's scan and top-k and running beside the top-k) returns bit for bit what the serial
    lagged schedule returns, eagerly and from a captured graph, on the FP8 / bf16 path."""
    cfg = production_config(D, layers=4)
    torch.manual_seed(21)
    model = D.DSAModel(cfg).eval().cuda().to(torch.bfloat16)
    B, S0, steps = 2, 300, 5
    prompt = torch.randn(B, S0, cfg.hidden_size, device="cuda").to(torch.bfloat16)
    toks = torch.randn(steps, B, cfg.hidden_size, device="cuda").to(torch.bfloat16)
    mode, cold = D.ScheduleMode.LAGGED_FUSED, D.ColdStartPolicy.EAGER

    def run(overlap, graph):
        st = model.init_decode(B, 320)
        assert st.fp8
        model.prefill(st, prompt, mode, cold)
        outs, sels = [], []
        if graph:
            g, x_in, x_out = model.capture_decode(st, mode, cold, overlap=overlap)
            for t in range(steps):
                x_in.copy_(toks[t])
                g.replay()
                outs.append(x_out.clone())
        else:
            for t in range(steps):
                rec = {}
                outs.append(model.decode_step(st, toks[t], mode, cold, overlap=overlap, record=rec).clone())
                sels.append([None if m is None else m.clone() for m in rec["produced"]])
        torch.cuda.synchronize()
        return torch.stack(outs), sels

    serial, sel_serial = run(False, False)
    chained, sel_chained = run("chained", False)
    graphed, _ = run("chained", True)
    assert torch.equal(serial, chained)
    assert torch.equal(serial, graphed)
    for a, b in zip(sel_serial, sel_chained):
        for ia, ib in zip(a, b):
            assert (ia is None) == (ib is None)
            if ia is not None:
                assert torch.equal(ia, ib)
    with pytest.raises(ValueError):
        st = model.init_decode(B, 320)
        model.decode_step(st, toks[0], mode, cold, overlap="chained", lag_depth=2)
    from dsa_multi_layer_indexer_b200 import _lib
    _lib.check_device_status()


def test_full_dimensions_decode_against_the_reference_model(D):
    """Two layers with the full-size dimensions (hidden 7168, 128 MLA heads, q_lora 1536,
    kv_lora 512, indexer 64 x 128, MLP 18432) under the lagged schedule: the bf16 / FP8 decode
    path (cuBLAS projections, dsa_decode_prep, FP8 scan, top-k, split-K attention) against what
    the reference's own fp32 DSAModel computed on the CPU from the same seed, with the same
    bf16-rounded weights (tests/golden/model_full_dims.npz). 160 tokens are prefilled, the last
    8 are decoded one by one. Tolerances: final hidden state within 6e-2 (bf16 activations against
    fp32), selected sets overlapping by more than 0.8 on average (the cutoff of a 64-of-160
    selection moves with bf16 / e4m3 rounding of the indexer operands)."""
    g = load_golden("model_full_dims.npz")
    cfg = D.DSAConfig(num_hidden_layers=2, first_k_dense_replace=0, index_topk=64)
    torch.manual_seed(3)
    model = D.DSAModel(cfg).eval()  # on the CPU, in the reference's construction order: the same weights
    with torch.no_grad():
        for prm in model.parameters():
            prm.copy_(prm.to(torch.bfloat16).float())
    w_sum = sum(float(prm.double().sum()) for prm in model.parameters())
    assert w_sum == pytest.approx(float(g["w_sum"]), rel=1e-9), "seeded weights differ from the fixture's"
    model = model.to(torch.bfloat16).cuda()
    S, tail = int(g["S"]), int(g["tail"])
    torch.manual_seed(3003)
    x = torch.randn(1, S, cfg.hidden_size).to(torch.bfloat16)
    assert float(x.float().double().sum()) == pytest.approx(float(g["x_sum"]), rel=1e-9)
    mode, cold = D.ScheduleMode.LAGGED_FUSED, D.ColdStartPolicy.EAGER
    st = model.init_decode(1, S + 8)
    assert st.fp8
    model.prefill(st, x[:, :S - tail].cuda(), mode, cold)
    ref_h = torch.from_numpy(g["hidden_tail"])
    overlaps, errs = [], []
    for t in range(tail):
        rec = {}
        h = model.decode_step(st, x[:, S - tail + t].cuda(), mode, cold, record=rec)
        errs.append(rel_err(h.float().cpu()[0], ref_h[t]))
        for kind in ("used", "produced"):
            for li, ours in enumerate(rec[kind]):
                name = f"{kind}_{li}"
                assert (ours is None) == (name not in g.files), name
                if ours is not None:
                    sa = set(int(v) for v in ours[0].tolist() if v >= 0)
                    sb = set(int(v) for v in g[name][t].tolist() if 0 <= v < S)
                    overlaps.append(len(sa & sb) / max(1, len(sa | sb)))
    assert max(errs) < 6e-2, errs
    assert min(overlaps) > 0.6 and sum(overlaps) / len(overlaps) > 0.8, overlaps
    del model
    torch.cuda.empty_cache()


def test_fused_decode_prep_matches_the_unfused_chain(D):
    """dsa_decode_prep (one launch) against the same chain written with torch ops in
    fp32: RoPE, per-head e4m3 quantisation with folded scales, both cache appends
    and the assembled absorbed query."""
    from dsa_multi_layer_indexer_b200 import ops
    from dsa_multi_layer_indexer_b200.rope import apply_rotary_at, build_rope_cache
    from oracle import dsa_oracle as O

    torch.manual_seed(21)
    B, H, Hidx, cap = 3, 32, 64, 300
    dev, bf = "cuda", torch.bfloat16
    iq_raw = torch.randn(B, Hidx, 128, device=dev).to(bf)
    w_raw = torch.randn(B, Hidx, device=dev).to(bf)
    ik_raw = torch.randn(B, 128, device=dev).to(bf)
    kv_a = torch.randn(B, 576, device=dev).to(bf)
    q = torch.randn(B, H, 192, device=dev).to(bf)
    q_abs = torch.randn(B, H, 512, device=dev).to(bf)
    norm_w = (1 + 0.1 * torch.randn(512, device=dev)).to(bf)
    pos = torch.tensor([5, 299, 0], device=dev)
    for interleave in (False, True):
        mc, ms = build_rope_cache(cap, 64, 10000.0, dev, bf)
        ic, isn = build_rope_cache(cap, 128, 10000.0, dev, bf, interleave=interleave)
        index_q = torch.zeros(B, Hidx, 128, dtype=torch.uint8, device=dev)
        index_w = torch.zeros(B, Hidx, device=dev)
        q_full = torch.zeros(B, H, 576, dtype=bf, device=dev)
        c_ik = torch.zeros(B, cap, 128, dtype=torch.uint8, device=dev)
        c_sk = torch.zeros(B, cap, device=dev)
        c_kv = torch.zeros(B, cap, 576, dtype=bf, device=dev)
        ops.decode_prep(iq_raw, w_raw, ik_raw, kv_a, q_abs, q[..., 128:], norm_w, mc, ms, ic, isn, pos, index_q,
                        index_w, q_full, c_ik, c_sk, c_kv, interleave, 1e-6)
        torch.cuda.synchronize()
        f = torch.float32
        # indexer query heads
        iq = apply_rotary_at(iq_raw.to(f), ic.to(f), isn.to(f), pos, interleave=interleave).cpu()
        iq8, sq = O.quantize_e4m3_rowwise(iq)
        got = O.e4m3_to_f32(index_q.cpu()) * (index_w.cpu() / w_raw.float().cpu()).unsqueeze(-1)
        want = O.e4m3_to_f32(iq8) * sq.unsqueeze(-1)
        assert rel_err(got, want) < 2e-2  # one e4m3 step at most where a rounding boundary is crossed
        assert torch.allclose(index_w.cpu(), sq * w_raw.float().cpu(), rtol=1e-5, atol=1e-7)
        # appended index key
        ik = apply_rotary_at(ik_raw.to(f), ic.to(f), isn.to(f), pos, interleave=interleave).cpu()
        ik8, sk = O.quantize_e4m3_rowwise(ik)
        bi = torch.arange(B)
        assert torch.allclose(c_sk.cpu()[bi, pos.cpu()], sk, rtol=1e-5)
        assert rel_err(O.e4m3_to_f32(c_ik.cpu()[bi, pos.cpu()]) * sk[:, None], O.e4m3_to_f32(ik8) * sk[:, None]) < 2e-2
        assert int(c_ik.sum()) == int(c_ik[bi.to(dev), pos].sum())  # nothing else was written
        # appended latent row
        ckv = kv_a[:, :512].to(f)
        normed = ckv * torch.rsqrt(ckv.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.to(f)
        krope = apply_rotary_at(kv_a[:, 512:].to(f), mc.to(f), ms.to(f), pos)
        want_row = torch.cat([normed, krope], -1)
        assert rel_err(c_kv[bi.to(dev), pos].float().cpu(), want_row.cpu()) < 1e-2
        # assembled query
        qr = apply_rotary_at(q[..., 128:].to(f), mc.to(f), ms.to(f), pos)
        assert torch.equal(q_full[..., :512], q_abs)
        assert rel_err(q_full[..., 512:].float().cpu(), qr.cpu()) < 1e-2


def test_library_rmsnorm_matches_torch(D):
    from dsa_multi_layer_indexer_b200 import ops

    torch.manual_seed(22)
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        x = torch.randn(5, 7168, device="cuda").to(dt)
        w = (1 + 0.1 * torch.randn(7168, device="cuda")).to(dt)
        xf = x.float()
        want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(dt)
        got = ops.rmsnorm(x, w, 1e-6)
        assert rel_err(got.float().cpu(), want.float().cpu()) < tol


@pytest.mark.parametrize("rows,dim", [(1, 7168), (3, 1536), (2, 512), (5, 8192), (1, 264)])
def test_fused_add_rmsnorm_and_silu_mul_match_torch_bitwise(D, rows, dim):
    """The fused residual-add + RMSNorm and SiLU * up round exactly like the separate torch
    operations they replace in the decode step."""
    from dsa_multi_layer_indexer_b200 import ops

    torch.manual_seed(dim)
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    d = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
    s, normed = ops.add_rmsnorm(x, d, w, 1e-6)
    s_ref = x + d
    assert torch.equal(s, s_ref)
    sf = s_ref.float()
    ref = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(torch.bfloat16)
    assert (normed.float() - ref.float()).abs().max() <= 2 ** -7 * ref.float().abs().max()
    assert torch.equal(normed, ops.rmsnorm(s_ref, w, 1e-6))  # same arithmetic as the plain norm
    g = torch.randn(rows, dim, device="cuda").to(torch.bfloat16) * 3
    u = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    got = ops.silu_mul(g, u)
    ref = torch.nn.functional.silu(g) * u
    assert (got.float() - ref.float()).abs().max() <= 2 ** -7 * ref.float().abs().max()
    odd = ops.silu_mul(g.flatten()[:dim - 3].clone(), u.flatten()[:dim - 3].clone()) if dim % 8 == 0 else None
    if odd is not None:  # a length that is not a multiple of 8 takes the scalar tail
        assert torch.equal(odd, got.flatten()[:dim - 3])


def test_stacked_decode_projections_share_storage_and_agree(D):
    """init_decode stacks the six small projections into two GEMVs: the parameters are
    views of the stacked weights (same state_dict, no copy), a state_dict load lands in
    the stacked storage, and the decode step agrees with the six separate GEMVs."""
    cfg = production_config(D, layers=2)
    torch.manual_seed(3)
    model = D.DSAModel(cfg).to(torch.bfloat16).eval().cuda()
    before = {k: v.clone() for k, v in model.state_dict().items()}
    hid = cfg.hidden_size
    prompt = torch.randn(1, 40, hid, device="cuda").to(torch.bfloat16)
    tok = torch.randn(1, hid, device="cuda").to(torch.bfloat16)

    def step(m):
        st = m.init_decode(1, 64, fp8=True)
        m.prefill(st, prompt)
        return m.decode_step(st, tok, D.ScheduleMode.BASELINE).float()

    layer = model.layers[0]
    assert not layer._stacked()
    out = step(model)  # init_decode stacks
    assert layer._stacked()
    assert layer.kv_a_proj.weight.data_ptr() == layer._wx[cfg.q_lora_rank:].data_ptr()
    after = model.state_dict()
    assert all(torch.equal(before[k], after[k]) for k in before)
    # loading weights writes through the views into the stacked tensors
    other = D.DSAModel(cfg).to(torch.bfloat16).eval().cuda()
    model.load_state_dict(other.state_dict())
    assert layer._stacked() and torch.equal(layer._wc[:layer.q_b_proj.weight.shape[0]], other.layers[0].q_b_proj.weight)
    model.load_state_dict(before)
    # moving / casting the module drops the stacking and the six-GEMV path gives the same answer
    plain = D.DSAModel(cfg).to(torch.bfloat16).eval().cuda()
    plain.load_state_dict(before)
    for l in plain.layers:
        l.fuse_decode_weights = lambda: None  # keep this copy unstacked
    ref = step(plain)
    assert not plain.layers[0]._stacked()
    assert rel_err(out.cpu(), ref.cpu()) < 2e-2


@pytest.mark.parametrize("b,n,k", [(1, 2240, 7168), (2, 515, 1536), (4, 64, 264), (3, 7, 8), (1, 4099, 4096)])
def test_skinny_gemv_matches_fp32_reference(D, b, n, k):
    from dsa_multi_layer_indexer_b200 import ops

    torch.manual_seed(n + k)
    x = torch.randn(b, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    got = ops.gemv(x, w)
    assert got.shape == (b, n) and got.dtype == torch.bfloat16
    ref = x.float() @ w.float().T
    assert (got.float() - ref).abs().max() <= 2 ** -7 * ref.abs().max() + 1e-3
    # a strided x (rows of a wider matrix) is accepted
    wide = torch.randn(b, k + 64, device="cuda").to(torch.bfloat16)
    assert torch.equal(ops.gemv(wide[:, :k], w), ops.gemv(wide[:, :k].contiguous(), w))
    with pytest.raises(ValueError):
        ops.gemv(torch.zeros(5, k, device="cuda", dtype=torch.bfloat16), w)
