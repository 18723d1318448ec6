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
class AttentionNames:
    """Tensor names of an attention layer, after the spec's prefix.  An architecture whose checkpoint
    names them otherwise passes its own table; the part knows no name by itself."""
    q: str = "q_proj"
    k: str = "k_proj"
    v: str = "v_proj"
    o: str = "o_proj"
    weight: str = ".weight"
    bias: str = ".bias"


@dataclass(frozen=True)
class SwiGluNames:
    """Tensor names of a SwiGLU MLP, after its prefix."""
    gate: str = "gate_proj.weight"
    up: str = "up_proj.weight"
    down: str = "down_proj.weight"


@dataclass(frozen=True)
class MoeNames:
    """Tensor names of a sparse block, after the spec's prefix; ``expert`` is a template over the expert's index."""
    router: str = "gate.weight"
    shared_gate: str = "shared_expert_gate.weight"
    shared: str = "shared_expert."
    expert: str = "experts.{e}."
    mlp: SwiGluNames = SwiGluNames()


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
    names: AttentionNames = AttentionNames()


@dataclass(frozen=True)
class DenseFfnSpec:
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "swiglu"
    names: SwiGluNames = SwiGluNames()


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
    names: MoeNames = MoeNames()


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
    # the two ends of the model, as far as they are more than a lookup and a product:
    embed_scale: float = 1.0                 # the table's rows are multiplied by this as they enter the residual stream
    logit_softcap: Optional[float] = None    # logits = cap * tanh(logits / cap)
    tied_head_name: Optional[str] = None     # with head_weight None: a checkpoint may still carry the head under this name
