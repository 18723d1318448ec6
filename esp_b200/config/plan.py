"""Architecture-neutral description of a decoder: what the engine builds from.

An architecture's typed configuration turns its own config.json keys into a
``ModelPlan``.  The plan names, layer by layer, which mixer, feed-forward, norm
and position encoding a block has and with which sizes and constants; the
engine looks each ``kind`` up in the part registries and never asks which
architecture it is running.  The order in which layers run is data as well
(``schedule``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class NormSpec:
    kind: str            # registry key, e.g. "rmsnorm"
    width: int
    eps: float
    weight: str          # tensor name of the scale vector


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # e.g. "rope_split_half"
    rotary_dim: int
    theta: float
    max_positions: int


@dataclass(frozen=True)
class AttentionSpec:
    """Softmax attention over cached keys and values with grouped query heads."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qkv_bias: bool
    out_bias: bool
    window: Optional[int]            # None: every earlier key; W: the query and W-1 predecessors
    position: Optional[PositionSpec]
    prefix: str                      # tensor-name prefix, e.g. "model.layers.3.self_attn."
    kind: str = "attention"


@dataclass(frozen=True)
class DenseFfnSpec:
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "swiglu"


@dataclass(frozen=True)
class MoeFfnSpec:
    """Softmax router, top-k routed SwiGLU experts, one shared SwiGLU expert
    scaled by a sigmoid gate."""
    hidden: int
    num_experts: int
    top_k: int
    norm_topk: bool
    expert_intermediate: int
    shared_intermediate: int
    prefix: str
    kind: str = "moe_swiglu_shared"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts it has and how they are arranged."""
    mixer: Any                       # any spec object with a ``kind``
    ffn: Any
    mixer_norm: NormSpec
    ffn_norm: NormSpec
    kind: str = "prenorm_residual"   # x += mixer(norm(x)); x += ffn(norm(x))


@dataclass(frozen=True)
class ScheduleEntry:
    """One call of a layer.  ``cache_of`` names an earlier schedule index whose
    cache this call reads instead of holding one of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelPlan:
    architecture: str
    hidden: int
    vocab: int
    max_positions: int
    blocks: list
    schedule: list
    final_norm: NormSpec
    embed_weight: str
    head_weight: Optional[str]       # None: the head is the embedding table
    stop_token_ids: tuple = ()
    # tensor names that a checkpoint may hold although nothing reads them
    tolerated_suffixes: tuple = ()
    extra: dict = field(default_factory=dict)
