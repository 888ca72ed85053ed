"""The configuration types the model classes read: the fields of ``minisgl.models.config`` (models/config.py:9-25,
:91-110) that the integer path uses.  The reference's own ``ModelConfig`` (built by ``from_hf``) can be passed
wherever these are expected: only the attributes below are read."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class RotaryConfig:
    head_dim: int
    rotary_dim: int
    max_position: int
    base: float
    scaling: Optional[Dict[str, Any]] = None
    apply_hadamard: bool = True


@dataclass(frozen=True)
class HadamardTransformConfig:
    enabled: bool = False
    block_size: int = 0
    targets: Tuple[str, ...] = ()
    r3_enabled: bool = False


@dataclass(frozen=True)
class ModelConfig:
    num_layers: int
    num_qo_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int
    vocab_size: int
    intermediate_size: int
    rms_norm_eps: float
    rotary_config: RotaryConfig
    tie_word_embeddings: bool = False
    hadamard_transform: HadamardTransformConfig = field(default_factory=HadamardTransformConfig)
