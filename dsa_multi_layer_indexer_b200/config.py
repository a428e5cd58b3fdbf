"""Model geometry and schedule enums for the B200 DSA decode path.

The field names, defaults, presets and enum values are the public contract of
the reference's ``src/lagged_indexer_dsa/config.py`` (``DSAConfig`` :77-155,
``AttentionType`` :14-26, ``ColdStartPolicy`` :43-57, ``ScheduleMode`` :60-74,
presets :162-197, ``named_config`` :200-210), so a config object or a
``state_dict`` built for one implementation loads in the other.
"""

from __future__ import annotations

import dataclasses
import enum
from typing import Optional, Tuple


class AttentionType(str, enum.Enum):
    """Kind of attention a layer runs: dense causal, or top-k sparse (DSA)."""

    FULL = "full"
    DSA = "dsa"


class ColdStartPolicy(str, enum.Enum):
    """What a DSA layer at depth 0 attends when no earlier indexer exists.

    DENSE attends every causal key; EAGER runs the layer's own indexer first
    and attends its selection (no lag for that one layer).
    """

    DENSE = "dense"
    EAGER = "eager"


class ScheduleMode(str, enum.Enum):
    """BASELINE: layer l attends layer l's own selection.
    LAGGED_REFERENCE / LAGGED_FUSED: layer l attends layer l-1's selection;
    the two differ only in whether the query latent is computed once (fused)
    or once per consumer (reference). On the GPU the lagged modes additionally
    let the indexer run on a second stream beside attention + MLP.
    """

    BASELINE = "baseline"
    LAGGED_REFERENCE = "lagged_reference"
    LAGGED_FUSED = "lagged_fused"


def dense_prefix_attention_types(num_hidden_layers: int, num_dense: int) -> Tuple[AttentionType, ...]:
    """``num_dense`` FULL layers followed by DSA layers (reference config.py:29-40)."""
    if num_dense < 0 or num_dense > num_hidden_layers:
        raise ValueError(f"num_dense must be in [0, {num_hidden_layers}], got {num_dense}")
    head = (AttentionType.FULL,) * num_dense
    tail = (AttentionType.DSA,) * (num_hidden_layers - num_dense)
    return head + tail


@dataclasses.dataclass(frozen=True)
class DSAConfig:
    """Dimensions of a stack of DSA blocks; defaults are DeepSeek-V3.2."""

    hidden_size: int = 7168
    num_hidden_layers: int = 61
    num_attention_heads: int = 128
    # multi-head latent attention
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    # lightning indexer
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 2048
    # feed-forward
    intermediate_size: int = 18432
    first_k_dense_replace: int = 3
    attention_layer_types: Optional[Tuple[AttentionType, ...]] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    indexer_rope_interleave: bool = False

    @property
    def qk_head_dim(self) -> int:
        """Width of one latent cache row in the absorbed MQA form (512 + 64 = 576)."""
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def resolved_attention_types(self) -> Tuple[AttentionType, ...]:
        if self.attention_layer_types is None:
            return (AttentionType.DSA,) * self.num_hidden_layers
        return tuple(AttentionType(t) for t in self.attention_layer_types)

    def __post_init__(self) -> None:
        n = self.num_hidden_layers
        if self.first_k_dense_replace < 0 or self.first_k_dense_replace > n:
            raise ValueError(
                f"first_k_dense_replace must be in [0, {n}], got {self.first_k_dense_replace}"
            )
        if self.index_topk <= 0:
            raise ValueError("index_topk must be positive")
        if self.num_attention_heads <= 0:
            raise ValueError("num_attention_heads must be positive")
        for name in ("qk_rope_head_dim", "index_head_dim"):
            if getattr(self, name) % 2:
                raise ValueError(f"{name} must be even for rotary embeddings")
        if self.attention_layer_types is not None:
            kinds = self.resolved_attention_types
            if len(kinds) != n:
                raise ValueError(
                    f"attention_layer_types has length {len(kinds)}, expected num_hidden_layers={n}"
                )

    @property
    def is_production_geometry(self) -> bool:
        """True when the tensor-core kernels apply: 576-wide latent rows with a
        512-wide value part, 128-wide index keys and at most 64 indexer heads in
        multiples of 16 (the same compile-time limits as the reference kernel,
        kernels/cuda_fused_sparse_splitk.py:53-55, :2498-2499)."""
        return (
            self.kv_lora_rank == 512
            and self.qk_rope_head_dim == 64
            and self.index_head_dim == 128
            and self.index_n_heads % 16 == 0
            and self.index_n_heads <= 64
        )


GLM5_CONFIG = DSAConfig(
    hidden_size=6144,
    num_hidden_layers=78,
    num_attention_heads=64,
    q_lora_rank=2048,
    kv_lora_rank=512,
    qk_nope_head_dim=192,
    qk_rope_head_dim=64,
    v_head_dim=256,
    index_n_heads=32,
    index_head_dim=128,
    index_topk=2048,
    intermediate_size=12288,
    first_k_dense_replace=3,
    rope_theta=1_000_000.0,
    indexer_rope_interleave=True,
)
GLM5_1_CONFIG = GLM5_CONFIG

SMALL_CONFIG = DSAConfig(
    hidden_size=256,
    num_hidden_layers=6,
    num_attention_heads=8,
    q_lora_rank=96,
    kv_lora_rank=64,
    qk_nope_head_dim=32,
    qk_rope_head_dim=16,
    v_head_dim=32,
    index_n_heads=8,
    index_head_dim=16,
    index_topk=16,
    intermediate_size=512,
)

_PRESETS = {
    "deepseek": DSAConfig(),
    "glm5": GLM5_CONFIG,
    "glm5.1": GLM5_1_CONFIG,
    "small": SMALL_CONFIG,
}


def named_config(name: str) -> DSAConfig:
    """Preset lookup by the names the reference accepts (config.py:200-210)."""
    try:
        return _PRESETS[name]
    except KeyError:
        raise ValueError(f"unknown config '{name}'; choose from {sorted(_PRESETS)}") from None
