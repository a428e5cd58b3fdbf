"""CPU oracle for the DSA decode hot path. TEST INFRASTRUCTURE, NOT PRODUCT.

A restatement, in plain torch-CPU / numpy, of the reference's algorithm for the
indexer scan, the top-k selection, the sparse MLA decode, the split-K merge, the
FP8 formats and the lagged schedule. Every function names the reference lines
it follows. Only tests, the smoke check and the bench's CPU-baseline leg may
import this module; the product package never does.

Parity status: PINNED. ``tests/golden/`` holds outputs of the reference's own
functions (imported from its source tree by ``tests/golden/make_golden.py``) on
seeded inputs, and ``tests/test_oracle_golden.py`` checks this module against
them, so the oracle travels to machines where the reference is absent.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

E4M3_MAX = 448.0


# ----------------------------------------------------------------------- FP8 e4m3
def e4m3_table() -> np.ndarray:
    """All 256 e4m3fn values as float32, built from the format definition
    (1 sign, 4 exponent bits with bias 7, 3 mantissa bits, no infinities,
    S.1111.111 = NaN). The reference relies on torch's float8_e4m3fn cast
    (kernels/cuda_fused_sparse_splitk.py:2969-2974); the tests check this table
    against that cast."""
    out = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = sign * (m / 8.0) * 2.0 ** (-6)
        else:
            v = sign * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = v
    return out


_E4M3 = torch.from_numpy(e4m3_table())


def e4m3_to_f32(bytes_u8: torch.Tensor) -> torch.Tensor:
    """Decode e4m3 bytes (uint8 or float8_e4m3fn tensor) to float32 exactly."""
    if bytes_u8.dtype == torch.float8_e4m3fn:
        bytes_u8 = bytes_u8.view(torch.uint8)
    return _E4M3[bytes_u8.long()]


def quantize_e4m3_rowwise(x: torch.Tensor, clamp_min: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric e4m3 quantisation -> (uint8 bytes, fp32 scale).
    Follows quantize_e4m3_rowwise, kernels/cuda_fused_sparse_splitk.py:2969-2974:
    amax clamped at 1e-6, scale = amax / 448, round-to-nearest-even cast."""
    x = x.float()
    amax = x.abs().amax(dim=-1, keepdim=True).clamp_min(clamp_min)
    scale = amax / E4M3_MAX
    q = (x / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale.squeeze(-1)


def make_fp8_indexer_inputs(iq: torch.Tensor, ik: torch.Tensor, w: torch.Tensor):
    """(iq8, ik8, w_folded, k_scale): the operand form the scan consumes, with
    the per-(row, head) query scale folded into the head weights. Follows
    make_fp8_indexer_inputs, kernels/cuda_fused_sparse_splitk.py:2977-2987
    (which draws its own randn; here the caller supplies iq [S,H,D], ik [N,D],
    w [S,H])."""
    iq8, sq = quantize_e4m3_rowwise(iq)
    ik8, sk = quantize_e4m3_rowwise(ik)
    return iq8.contiguous(), ik8.contiguous(), (sq * w.float()).contiguous(), sk.contiguous()


# ----------------------------------------------------------------------- a1 indexer
def indexer_logits_f32(index_q: torch.Tensor, index_k: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """I[b,t,s] = sum_h w[b,t,h] relu(q[b,t,h].k[b,s]).
    Follows indexer_logits, src/lagged_indexer_dsa/attention_core.py:27-49.
    index_q [B,S,H,D], index_k [B,N,D], weights [B,S,H] -> [B,S,N]."""
    score = torch.einsum("bshd,bnd->bshn", index_q.float(), index_k.float())
    return (torch.relu(score) * weights.float().unsqueeze(-1)).sum(dim=2)


def indexer_logits_fp8(iq8: torch.Tensor, ik8: torch.Tensor, w_folded: torch.Tensor, k_scale: torch.Tensor,
                       chunk: int = 16384) -> torch.Tensor:
    """Logits from the same e4m3 bytes the GPU reads: [S,H,D] x [N,D] -> [S,N].
    Follows ref_indexer_logits_fp8, kernels/cuda_fused_sparse_splitk.py:2990-2992
    (decode to fp32, bilinear, relu, weighted head sum, per-key scale); keys are
    processed in chunks only to bound memory."""
    q = e4m3_to_f32(iq8)
    out = torch.empty(q.shape[0], ik8.shape[0], dtype=torch.float32)
    for s0 in range(0, ik8.shape[0], chunk):
        k = e4m3_to_f32(ik8[s0:s0 + chunk])
        bil = torch.einsum("shd,gd->shg", q, k)
        out[:, s0:s0 + chunk] = (bil.relu() * w_folded.float().unsqueeze(-1)).sum(1) * k_scale[s0:s0 + chunk].view(1, -1)
    return out


def mask_beyond(logits: torch.Tensor, seq_lens: Sequence[int]) -> torch.Tensor:
    """-inf for key positions >= seq_lens[row]: the decode form of the causal gate
    (kernel `g <= q_pos`, kernels/cuda_fused_sparse_splitk.py:627, :1702-1711;
    full-sequence form apply_causal_mask, attention_core.py:52-63)."""
    out = logits.clone()
    pos = torch.arange(logits.shape[-1])
    for r, n in enumerate(seq_lens):
        out[r, pos >= int(n)] = float("-inf")
    return out


# ----------------------------------------------------------------------- a3 top-k
def select_topk(logits: torch.Tensor, topk: int, pad_value: int) -> torch.Tensor:
    """Positions of the top-k finite logits per row, as a SORTED int64 [R, topk]
    padded with ``pad_value``. Set semantics of select_topk,
    src/lagged_indexer_dsa/attention_core.py:66-91 (non-finite values become the
    sentinel, short rows are padded); ties are resolved toward the lower
    position (the kernels' convention, kernels/cuda_fused_sparse_splitk.py:919-921),
    which torch.topk leaves unspecified."""
    R, n = logits.shape
    out = torch.full((R, topk), pad_value, dtype=torch.int64)
    for r in range(R):
        row = logits[r].double()
        order = torch.sort(row, descending=True, stable=True).indices  # stable: lower index first among ties
        take = order[: min(topk, n)]
        take = take[torch.isfinite(row[take])]
        take = torch.sort(take).values
        out[r, : take.numel()] = take
    return out


# ----------------------------------------------------------------------- a4 sparse MLA
def sparse_mla_decode(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, seq_lens: Sequence[int],
                      sm_scale: float, value_dim: int = 512) -> torch.Tensor:
    """out[r,h] = softmax_j(scale q[r,h].kv[idx_j]) . kv[idx_j,:value_dim] over
    the entries 0 <= idx < seq_lens[r]. q [R,H,D], kv [N,D] (shared by all rows),
    indices [R,topk]. Follows ref_sparse_mla, kernels/cuda_fused_sparse_splitk.py
    :2950-2966 (q_pos = seq_len - 1), equivalently _selection_mask + _attend,
    attention_core.py:94-118. fp32 math on the given values."""
    R, H, _ = q.shape
    out = torch.zeros(R, H, value_dim, dtype=torch.float32)
    kvf = kv.float()
    for r in range(R):
        idx = indices[r].long()
        sel = idx[(idx >= 0) & (idx < int(seq_lens[r]))]
        if sel.numel() == 0:
            continue
        k = kvf[sel]
        p = torch.softmax((q[r].float() @ k.t()) * sm_scale, dim=-1)
        out[r] = p @ k[:, :value_dim]
    return out


def dense_mla_decode(q: torch.Tensor, kv: torch.Tensor, seq_lens: Sequence[int], sm_scale: float,
                     value_dim: int = 512) -> torch.Tensor:
    """Dense causal attention of the cold start (dense_mla_core, attention_core.py:149-160)."""
    R = q.shape[0]
    idx = torch.arange(kv.shape[0]).unsqueeze(0).expand(R, -1)
    return sparse_mla_decode(q, kv, idx, seq_lens, sm_scale, value_dim)


def splitk_merge(acc: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """Log-sum-exp merge of split partials: acc [S,H,V] unnormalised, m/l [S,H]
    (m in base-2 exponent units). Follows combine_kernel,
    kernels/cuda_fused_sparse_splitk.py:996-1045 including the -inf skip."""
    mx = m.max(dim=0).values
    e = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), torch.exp2(m - mx))
    lsum = (l * e).sum(0)
    o = (acc * e.unsqueeze(-1)).sum(0)
    return torch.where(lsum.unsqueeze(-1) > 0, o / lsum.unsqueeze(-1).clamp_min(1e-38), torch.zeros_like(o))


# ----------------------------------------------------------------------- FP8 latent rows
def pack_fp8_latent(kv: torch.Tensor) -> torch.Tensor:
    """[N,576] -> [N,656] uint8 rows: 512 e4m3 | 4 fp32 scales (one per 128
    dims) | 64 bf16 rope. Layout of the serving pool,
    kernels/cuda_fused_sparse_splitk.py:1098-1104; scale = amax/448 per group."""
    n = kv.shape[0]
    nope = kv[:, :512].float().reshape(n, 4, 128)
    amax = nope.abs().amax(-1, keepdim=True).clamp_min(1e-4)
    scale = amax / E4M3_MAX
    q = (nope / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8).reshape(n, 512)
    rope = kv[:, 512:].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(n, 128)
    sc = scale.reshape(n, 4).contiguous().view(torch.uint8).reshape(n, 16)
    return torch.cat([q, sc, rope], dim=1).contiguous()


def unpack_fp8_latent(rows: torch.Tensor) -> torch.Tensor:
    """[N,656] uint8 -> [N,576] bf16 exactly as the kernels dequantise:
    fp8 -> f32, x group scale (f32), round to bf16
    (hp_dequant4, kernels/cuda_fused_sparse_splitk.py:1181-1196)."""
    n = rows.shape[0]
    vals = e4m3_to_f32(rows[:, :512]).reshape(n, 4, 128)
    scale = rows[:, 512:528].contiguous().view(torch.float32).reshape(n, 4, 1)
    nope = (vals * scale).to(torch.bfloat16).reshape(n, 512)
    rope = rows[:, 528:].contiguous().view(torch.bfloat16).reshape(n, 64)
    return torch.cat([nope, rope], dim=1)


# ----------------------------------------------------------------------- paged index keys
def pack_index_pages(ik8: torch.Tensor, k_scale: torch.Tensor, page_ids: Sequence[int], num_pages: int,
                     pool: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Scatter a sequence's e4m3 keys [N,128] + scales [N] into 64-token pages of
    8448 bytes ([64 x 128 B keys][64 x fp32 scales]); layout from
    kernels/cuda_fused_sparse_splitk.py:540-546, :2428-2429."""
    if pool is None:
        pool = torch.zeros(num_pages, 8448, dtype=torch.uint8)
    n = ik8.shape[0]
    for j, pid in enumerate(page_ids):
        lo, hi = j * 64, min(n, j * 64 + 64)
        if lo >= n:
            break
        page = pool[pid]
        page[: (hi - lo) * 128] = ik8[lo:hi].reshape(-1)
        sc = torch.zeros(64, dtype=torch.float32)
        sc[: hi - lo] = k_scale[lo:hi]
        page[8192:] = sc.view(torch.uint8)
    return pool


# ----------------------------------------------------------------------- inputs with a margin
def enforce_topk_margin(logits: torch.Tensor, k_scale: torch.Tensor, topk: int, band: float = 2e-2,
                        max_iter: int = 50) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rescale per-key scales so no logit lies within ``band * max|logit|`` of
    the rank-topk cutoff; the logit is linear in k_scale[s]
    (kernels/cuda_fused_sparse_splitk.py:630, :2992), so logits scale with it.
    Returns (new_scale, new_logits) for one row of logits [N]. With such inputs
    any implementation whose logits are within band/2 selects the same set."""
    logits = logits.clone().double()
    scale = k_scale.clone().double()
    for _ in range(max_iter):
        srt = torch.sort(logits, descending=True).values
        tau = 0.5 * (srt[topk - 1] + srt[topk])
        width = band * logits.abs().max()
        near = (logits - tau).abs() < width
        if not bool(near.any()):
            break
        above = near & (logits >= tau)
        below = near & (logits < tau)
        # push away from the cutoff multiplicatively (sign-aware)
        for sel, up in ((above, True), (below, False)):
            if bool(sel.any()):
                target = tau + (2.0 * width if up else -2.0 * width)
                lv = logits[sel]
                safe = lv.abs() > 1e-12
                f = torch.where(safe, target / torch.where(safe, lv, torch.ones_like(lv)), torch.ones_like(lv))
                f = torch.where(f > 0, f, torch.ones_like(f))
                scale[sel] = scale[sel] * f
                logits[sel] = lv * f
    return scale.float(), logits.float()


# ----------------------------------------------------------------------- a9 schedule
def lagged_producers(is_dsa: Sequence[bool]) -> List[bool]:
    """Layer L runs an indexer under the lagged schedule iff layer L+1 attends
    sparsely (src/lagged_indexer_dsa/model.py:61-71)."""
    n = len(is_dsa)
    return [(i + 1 < n and bool(is_dsa[i + 1])) for i in range(n)]


def schedule_plan(is_dsa: Sequence[bool], mode: str, cold_start: str) -> List[dict]:
    """Per layer: which selection attention consumes ('own', 'prev', 'dense') and
    whether the layer's indexer runs. Restates DSAModel.forward's control flow
    (src/lagged_indexer_dsa/model.py:93-136) without tensors."""
    plan = []
    prod = lagged_producers(is_dsa)
    for i, dsa in enumerate(is_dsa):
        if mode == "baseline":
            plan.append({"attend": "own" if dsa else "dense", "produce": bool(dsa)})
        else:
            if not dsa:
                attend = "dense"
            elif i == 0:
                attend = "dense" if cold_start == "dense" else "own"
            else:
                attend = "prev"
            plan.append({"attend": attend, "produce": prod[i]})
    return plan


def schedule_plan_depth(is_dsa: Sequence[bool], runs_indexer: Sequence[bool], cold_start: str,
                        depth: int) -> List[dict]:
    """Lag depth k >= 2 without tensors: per layer, whose fresh set the attention
    consumes (``("layer", j)``, or ``"dense"``) and whether the layer's indexer
    runs. Restates the documented semantics of the serving overlay's
    ``_hh_lag_refresh_dispatch_depth``
    (sglang_overlay/mli-sglang-v0.5.16.patch:3017-3100): FIFO of depth k of fresh
    sets; a refresh layer attends the oldest entry once the FIFO is full, else the
    incoming carry; its carry-out is the set it attended; skip layers copy the
    carry; the first sparse layer bootstraps (own set under "eager", dense
    attention with its set queued under "dense")."""
    plan, fifo, carried, booted = [], [], "dense", False
    for i, dsa in enumerate(is_dsa):
        if not dsa:
            plan.append({"attend": "dense", "produce": False})
            continue
        if not booted:
            booted = True
            if cold_start == "dense":
                attend, produce = "dense", bool(runs_indexer[i])
                if produce:
                    fifo.append(i)
            else:
                attend, produce = ("layer", i), True
            carried = attend
        elif runs_indexer[i]:
            attend = ("layer", fifo.pop(0)) if len(fifo) >= depth else carried
            fifo.append(i)
            carried, produce = attend, True
        else:
            attend, produce = carried, False
        plan.append({"attend": attend, "produce": produce})
    return plan


# ------------------------------------------------- serving-form indexer staging
def layer_norm_128(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """LayerNorm in fp32 with weight and bias, result in x's dtype
    (inference/modeling/transformer.py:418-433)."""
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight, bias, eps).type_as(x)


def rotary_embed(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """Rotary embedding as a complex product in fp32, result in x's dtype
    (inference/modeling/transformer.py:525-547). x [..., 2n]; cos / sin broadcast
    to [..., n] (real / imaginary part of freqs_cis). interleaved: the complex
    pair i is (x[2i], x[2i+1]); otherwise (x[i], x[i+n]) and the output keeps the
    real parts in the first half."""
    xf = x.float()
    n = x.shape[-1] // 2
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
    else:
        a, b = xf[..., :n], xf[..., n:]
    re = a * cos - b * sin
    im = a * sin + b * cos
    if interleaved:
        y = torch.stack([re, im], dim=-1).flatten(-2)
    else:
        y = torch.cat([re, im], dim=-1)
    return y.to(x.dtype)


def hadamard_rotate(x: torch.Tensor) -> torch.Tensor:
    """rotate_activation on its pure-torch path: bf16 input, Walsh-Hadamard
    butterfly in fp32 (strides 1, 2, ..., n/2; the element with the stride bit
    clear gets the sum, the other the difference), times n^-0.5, back to bf16
    (inference/modeling/transformer.py:550-568, :571-592)."""
    dtype = x.dtype
    n = x.shape[-1]
    v = x.to(torch.bfloat16).float().reshape(-1, n).clone()
    h = 1
    while h < n:
        w = v.view(-1, n // (2 * h), 2, h)
        even, odd = w[:, :, 0, :].clone(), w[:, :, 1, :].clone()
        w[:, :, 0, :] = even + odd
        w[:, :, 1, :] = even - odd
        h *= 2
    y = (v * (n ** -0.5)).view(x.shape).to(torch.bfloat16)
    return y.to(dtype)


def act_quant_128(x: torch.Tensor, round_scale: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """act_quant over blocks of 128 (inference/modeling/kernels.py:19-117), for a
    last dimension of exactly 128: amax = max(|x|, 1e-4) in fp32, scale =
    amax * (1/448) or, with a scale format, 2^ceil(log2(amax * (1/448))) by the
    reference's bit arithmetic (exponent + 1 when the mantissa is non-zero);
    y = e4m3(clamp(x / scale, -448, 448)). Returns (uint8 bytes, fp32 scale [..., 1])."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
    scale = amax * torch.tensor(1.0 / 448.0, dtype=torch.float32)
    if round_scale:
        bits = scale.view(torch.int32)
        e = ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)
        scale = ((e + 127) << 23).to(torch.int32).view(torch.float32)
    y = (xf / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    return y, scale


def indexer_stage_fp8(q_raw: torch.Tensor, k_raw: torch.Tensor, w_raw: torch.Tensor, norm_w: torch.Tensor,
                      norm_b: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
                      positions: Sequence[int], interleaved: bool, round_scale: bool,
                      softmax_scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Indexer.stage_fp8_operands after its three projections
    (inference/modeling/transformer.py:1044-1066): q_raw bf16 [B, H, 128],
    k_raw bf16 [B, 128], w_raw fp32 [B, H], cos / sin fp32 [cap, 32]. Returns
    (q bytes [B, H, 128], folded head weights [B, H], key bytes [B, 128], key
    scale [B])."""
    B, H, _ = q_raw.shape
    pos = torch.as_tensor(list(positions), dtype=torch.long)
    c, s = cos[pos], sin[pos]                                    # [B, 32]
    q = torch.cat([rotary_embed(q_raw[..., :64], c[:, None, :], s[:, None, :], interleaved), q_raw[..., 64:]], dim=-1)
    k = layer_norm_128(k_raw, norm_w, norm_b, eps)
    k = torch.cat([rotary_embed(k[..., :64], c, s, interleaved), k[..., 64:]], dim=-1)
    q, k = hadamard_rotate(q), hadamard_rotate(k)
    q8, q_scale = act_quant_128(q, round_scale)
    k8, k_scale = act_quant_128(k, round_scale)
    weights = w_raw.float() * (H ** -0.5)
    weights = (weights.unsqueeze(-1) * q_scale * softmax_scale).squeeze(-1)
    return q8, weights, k8, k_scale.squeeze(-1)


# --------------------------------------------------- serving-form latent append
def rms_norm_f32w(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of the serving model: fp32 math, fp32 weight, result in x's dtype
    (inference/modeling/transformer.py:380-410)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (weight * (xf * torch.rsqrt(var + eps))).to(x.dtype)


def latent_append_rows(kv_a: torch.Tensor, norm_w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
                       positions: Sequence[int], interleaved: bool, fmt: str, round_scale: bool) -> torch.Tensor:
    """The new token's latent row as the cache receives it
    (inference/modeling/transformer.py:3264-3276): kv_a bf16 [B, 576] = wkv_a(x);
    RMSNorm of dims 0..511, rotary embedding of dims 512..575. fmt "bf16": the row as
    it is; "bf16_quant": latent dims through act_quant and back (:3268-3274);
    "fp8": the 656-byte packed row (kernels/cuda_fused_sparse_splitk.py:1098-1104),
    uint8 [B, 656]."""
    pos = torch.as_tensor(list(positions), dtype=torch.long)
    kv = rms_norm_f32w(kv_a[:, :512], norm_w, eps)
    pe = rotary_embed(kv_a[:, 512:], cos[pos], sin[pos], interleaved)
    if fmt == "bf16":
        return torch.cat([kv, pe], dim=-1)
    B = kv.shape[0]
    y, scale = act_quant_128(kv.reshape(B, 4, 128), round_scale)
    if fmt == "bf16_quant":
        deq = (e4m3_to_f32(y) * scale).to(kv.dtype).reshape(B, 512)
        return torch.cat([deq, pe], dim=-1)
    rope = pe.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(B, 128)
    sc = scale.reshape(B, 4).contiguous().view(torch.uint8).reshape(B, 16)
    return torch.cat([y.reshape(B, 512), sc, rope], dim=1).contiguous()
