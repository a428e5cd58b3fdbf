"""Rotary position tables and their application (host-side preparation).

Two pairings of the head dimension exist and must be used consistently by the
table builder and by ``apply_rotary``: the half-split pairing ``(i, i + d/2)``
of DeepSeek-V3.2 and the adjacent pairing ``(2i, 2i + 1)`` of GLM-5. Same
contract as the reference's ``src/lagged_indexer_dsa/rope.py:25-84``. These run
as ordinary torch ops on whatever device the inputs live on; they are outside
the timed kernels.
"""

from __future__ import annotations

from typing import Tuple

import torch


def build_rope_cache(
    seq_len: int,
    head_dim: int,
    theta: float,
    device: torch.device,
    dtype: torch.dtype,
    interleave: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(cos, sin)`` tables of shape ``[seq_len, head_dim]``."""
    if head_dim % 2:
        raise ValueError("head_dim must be even for rotary embeddings")
    n_pairs = head_dim // 2
    exponent = torch.arange(n_pairs, device=device, dtype=torch.float32) / n_pairs
    inv_freq = 1.0 / (theta ** exponent)  # same rounding order as the reference (rope.py:41)
    angle = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv_freq[None, :]
    if interleave:
        full = angle.repeat_interleave(2, dim=1)
    else:
        full = torch.cat([angle, angle], dim=1)
    return torch.cos(full).to(dtype), torch.sin(full).to(dtype)


def _partner(x: torch.Tensor, interleave: bool) -> torch.Tensor:
    """The vector that multiplies ``sin``: each pair ``(a, b)`` becomes ``(-b, a)``."""
    if interleave:
        even, odd = x[..., 0::2], x[..., 1::2]
        return torch.stack([-odd, even], dim=-1).reshape(x.shape)
    lo, hi = x.chunk(2, dim=-1)
    return torch.cat([-hi, lo], dim=-1)


def apply_rotary(
    x: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    interleave: bool = False,
) -> torch.Tensor:
    """Rotate ``x[..., seq_len, head_dim]`` by the first ``seq_len`` table rows."""
    n = x.shape[-2]
    if cos.shape[-2] < n:
        raise ValueError(f"rope cache too short: have {cos.shape[-2]}, need {n}")
    c = cos[:n].to(x.dtype)
    s = sin[:n].to(x.dtype)
    return x * c + _partner(x, interleave) * s


def apply_rotary_at(
    x: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    positions: torch.Tensor,
    interleave: bool = False,
) -> torch.Tensor:
    """Decode form: rotate ``x[B, ..., head_dim]`` by table row ``positions[B]``.

    The reference layer has no decode entry; this is ``apply_rotary`` applied
    to one position per batch row, so that a decode step reproduces the last
    row of the full-sequence forward.
    """
    c = cos.index_select(0, positions).to(x.dtype)
    s = sin.index_select(0, positions).to(x.dtype)
    while c.dim() < x.dim():
        c = c.unsqueeze(1)
        s = s.unsqueeze(1)
    return x * c + _partner(x, interleave) * s
