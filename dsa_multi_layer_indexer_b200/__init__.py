"""B200-native (sm_100a) DSA decode hot path: lightning-indexer scan, exact
top-k selection, split-K sparse MLA decode and the multi-layer-indexer (MLI)
lagged schedule, behind the Python API of ``lagged_indexer_dsa``
(reference src/lagged_indexer_dsa/__init__.py:13-55).

All compute goes through libdsa_b200.so (C ABI in include/dsa_b200.h); there is
no CPU or torch-kernel fallback.
"""

from .config import (
    GLM5_1_CONFIG,
    GLM5_CONFIG,
    SMALL_CONFIG,
    AttentionType,
    ColdStartPolicy,
    DSAConfig,
    ScheduleMode,
    dense_prefix_attention_types,
    named_config,
)

from .dsa_layer import DSALayer, LayerDecodeCache, RopeCaches
from .model import DecodeState, DSAModel, ForwardTrace

__all__ = [
    "DSALayer",
    "RopeCaches",
    "LayerDecodeCache",
    "DSAModel",
    "ForwardTrace",
    "DecodeState",
    "GLM5_1_CONFIG",
    "GLM5_CONFIG",
    "SMALL_CONFIG",
    "AttentionType",
    "ColdStartPolicy",
    "DSAConfig",
    "ScheduleMode",
    "dense_prefix_attention_types",
    "named_config",
]
