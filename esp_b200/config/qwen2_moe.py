"""Typed configuration of the Qwen2 MoE decoder, read from its own config.json
keys with the reference's defaults, refusals and derived values
(crates/esp/src/infer/decoder/config.rs:36-51, :230-316, :322-386, :434-570).
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass, field
from typing import Optional

from ..errors import InvalidConfig, Unsupported
from .plan import (AttentionNames, AttentionSpec, BlockSpec, MoeNames, SwiGluNames, DenseFfnSpec, ModelPlan, MoeFfnSpec, NormSpec,
                   PositionSpec, ScheduleEntry)
from .registry import register_architecture

ARCHITECTURE = "Qwen2MoeForCausalLM"
MODEL_TYPE = "qwen2_moe"
_MAX_DIM = 1 << 40


def _f32(x: float) -> float:
    """The reference parses rope_theta as a 32-bit float and rms_norm_eps as a
    64-bit one (config.rs:351-354)."""
    return struct.unpack("<f", struct.pack("<f", float(x)))[0]


def _need_int(raw, key, default=None, required=True):
    v = raw.get(key, default)
    if v is None:
        if required:
            raise InvalidConfig(f"config.json lacks {key}")
        return None
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise InvalidConfig(f"{key} must be a non-negative integer, got {v!r}")
    return v


def _need_float(raw, key, default):
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise InvalidConfig(f"{key} must be a number, got {v!r}")
    return float(v)


def _need_bool(raw, key, default):
    v = raw.get(key, default)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise InvalidConfig(f"{key} must be true or false, got {v!r}")
    return v


@dataclass
class Qwen2MoeConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    max_position_embeddings: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    use_sliding_window: Optional[bool] = None
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[list] = None
    norm_topk_prob: bool = False
    decoder_sparse_step: int = 1
    mlp_only_layers: list = field(default_factory=list)
    eos_token_id: Optional[object] = None   # int, list of ints or absent (config.rs:361-378)

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2MoeConfig":
        cls._refuse_features(raw)
        sw = raw.get("sliding_window")
        if sw is not None and (isinstance(sw, bool) or not isinstance(sw, int) or sw < 0):
            raise InvalidConfig(f"sliding_window must be a non-negative integer or null, got {sw!r}")
        usw = raw.get("use_sliding_window")
        if usw is not None and not isinstance(usw, bool):
            raise InvalidConfig(f"use_sliding_window must be true, false or null, got {usw!r}")
        only = raw.get("mlp_only_layers", [])
        if only is None:
            only = []
        if not isinstance(only, list) or any(isinstance(i, bool) or not isinstance(i, int) or i < 0 for i in only):
            raise InvalidConfig("mlp_only_layers must be a list of layer indices")
        types = raw.get("layer_types")
        if types is not None and (not isinstance(types, list) or not all(isinstance(t, str) for t in types)):
            raise InvalidConfig("layer_types must be a list of strings")
        eos = raw.get("eos_token_id")
        if eos is not None:
            ok = (isinstance(eos, int) and not isinstance(eos, bool)) or (
                isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos))
            if not ok:
                raise InvalidConfig("eos_token_id must be an integer or a list of integers")
        cfg = cls(
            vocab_size=_need_int(raw, "vocab_size"),
            hidden_size=_need_int(raw, "hidden_size"),
            intermediate_size=_need_int(raw, "intermediate_size"),
            num_hidden_layers=_need_int(raw, "num_hidden_layers"),
            num_attention_heads=_need_int(raw, "num_attention_heads"),
            max_position_embeddings=_need_int(raw, "max_position_embeddings"),
            num_experts=_need_int(raw, "num_experts"),
            num_experts_per_tok=_need_int(raw, "num_experts_per_tok"),
            moe_intermediate_size=_need_int(raw, "moe_intermediate_size"),
            shared_expert_intermediate_size=_need_int(raw, "shared_expert_intermediate_size"),
            num_key_value_heads=_need_int(raw, "num_key_value_heads", required=False),
            head_dim=_need_int(raw, "head_dim", required=False),
            rms_norm_eps=_need_float(raw, "rms_norm_eps", 1e-5),
            rope_theta=_f32(_need_float(raw, "rope_theta", 10000.0)),
            tie_word_embeddings=_need_bool(raw, "tie_word_embeddings", False),
            use_sliding_window=usw,
            sliding_window=sw,
            max_window_layers=_need_int(raw, "max_window_layers", required=False),
            layer_types=types,
            norm_topk_prob=_need_bool(raw, "norm_topk_prob", False),
            decoder_sparse_step=_need_int(raw, "decoder_sparse_step", 1),
            mlp_only_layers=list(only),
            eos_token_id=eos,
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _refuse_features(raw: dict) -> None:
        """crates/esp/src/infer/decoder/config.rs:259-316, plus rope_scaling,
        which this library does not implement for any value but null."""
        for key in ("hidden_act", "hidden_activation"):
            act = raw.get(key)
            if act is not None and act not in ("silu", "swish"):
                raise Unsupported(key, f"{act!r}; only the SiLU-gated MLP is implemented")
        prf = raw.get("partial_rotary_factor")
        if prf is not None and prf != 1.0:
            raise Unsupported("partial_rotary_factor", f"{prf}; RoPE is applied to the full head")
        if raw.get("mlp_bias") is True:
            raise Unsupported("mlp_bias", "MLP projections are bias-free")
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            if raw.get(key) is not None:
                raise Unsupported(key, f"{raw[key]}; logit soft-capping is not implemented")
        for key in ("num_local_experts", "n_routed_experts"):
            n = raw.get(key)
            if isinstance(n, int) and n > 0:
                raise Unsupported(key, f"{n}; this architecture names its experts num_experts")
        if raw.get("rope_scaling") is not None:
            raise Unsupported("rope_scaling", f"{raw['rope_scaling']!r}; only unscaled rotary encoding is implemented")

    # ---- derived values (config.rs:434-490) -------------------------------
    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads if self.num_key_value_heads is not None else self.num_attention_heads

    @property
    def resolved_head_dim(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_attention_heads

    @property
    def query_width(self) -> int:
        return self.num_attention_heads * self.resolved_head_dim

    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.kv_heads

    # q/k/v always carry a bias and o_proj never does, whatever attention_bias
    # or qkv_bias say (config.rs:448-454)
    qkv_bias = True
    output_bias = False

    def layer_is_moe(self, index: int) -> bool:
        return index not in self.mlp_only_layers and (index + 1) % self.decoder_sparse_step == 0

    def layer_window(self, index: int) -> Optional[int]:
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[index] == "sliding_attention" else None
        if self.use_sliding_window is False:
            return None
        mwl = self.max_window_layers if self.max_window_layers is not None else 28
        if self.use_sliding_window is True and index >= mwl:
            return self.sliding_window
        return None

    def stop_token_ids(self) -> tuple:
        if self.eos_token_id is None:
            return ()
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(self.eos_token_id)

    # ---- validation (config.rs:492-570) ------------------------------------
    def validate(self) -> None:
        if self.num_attention_heads == 0 or (self.head_dim is None and self.hidden_size % self.num_attention_heads != 0):
            raise InvalidConfig(f"hidden_size {self.hidden_size} not divisible by num_attention_heads {self.num_attention_heads}")
        if self.kv_heads == 0 or self.num_attention_heads % self.kv_heads != 0:
            raise InvalidConfig(f"num_attention_heads {self.num_attention_heads} not divisible by num_key_value_heads {self.kv_heads}")
        hd = self.resolved_head_dim
        if hd == 0 or hd % 2 != 0:
            raise InvalidConfig(f"head_dim {hd} must be even for rotary encoding")
        bad = (self.hidden_size == 0 or self.intermediate_size == 0 or self.vocab_size == 0
               or self.num_hidden_layers == 0 or self.max_position_embeddings == 0
               or not math.isfinite(self.rms_norm_eps) or self.rms_norm_eps <= 0.0
               or not math.isfinite(self.rope_theta) or self.rope_theta <= 0.0
               or self.sliding_window == 0
               or self.num_attention_heads * hd >= _MAX_DIM or self.vocab_size * self.hidden_size >= _MAX_DIM)
        if bad:
            raise InvalidConfig("zero, non-finite or overflowing decoder dimensions/settings")
        if self.layer_types is not None:
            ok = len(self.layer_types) == self.num_hidden_layers and all(
                t in ("full_attention", "sliding_attention") for t in self.layer_types) and not (
                "sliding_attention" in self.layer_types and self.sliding_window is None)
            if not ok:
                raise Unsupported("layer_types", "expected one supported attention type per layer and a window for sliding layers")
        moe_bad = (self.num_experts == 0 or self.num_experts_per_tok == 0
                   or self.num_experts_per_tok > self.num_experts
                   or self.moe_intermediate_size == 0 or self.shared_expert_intermediate_size == 0
                   or self.decoder_sparse_step == 0
                   or any(i >= self.num_hidden_layers for i in self.mlp_only_layers)
                   or self.num_experts * self.moe_intermediate_size * self.hidden_size >= _MAX_DIM)
        if moe_bad:
            raise Unsupported("experts", "invalid expert count, routing, intermediate size or sparse-layer selection")

    # ---- writing ------------------------------------------------------------
    def to_dict(self) -> dict:
        d = {"architectures": [ARCHITECTURE], "model_type": MODEL_TYPE, "hidden_act": "silu"}
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "max_position_embeddings", "rms_norm_eps", "rope_theta",
                  "tie_word_embeddings", "use_sliding_window", "sliding_window", "max_window_layers", "layer_types",
                  "num_experts", "num_experts_per_tok", "norm_topk_prob", "moe_intermediate_size",
                  "shared_expert_intermediate_size", "decoder_sparse_step", "mlp_only_layers", "eos_token_id"):
            v = getattr(self, k)
            if v is not None:
                d[k] = v
        return d

    # ---- the plan the engine builds from --------------------------------------
    def plan(self) -> ModelPlan:
        hd = self.resolved_head_dim
        pos = PositionSpec("rope_split_half", hd, self.rope_theta, self.max_position_embeddings)
        blocks = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            mixer = AttentionSpec(self.hidden_size, self.num_attention_heads, self.kv_heads, hd,
                                  self.qkv_bias, self.output_bias, self.layer_window(i), pos, p + "self_attn.",
                                  names=ATTENTION_NAMES)
            if self.layer_is_moe(i):
                ffn = MoeFfnSpec(self.hidden_size, self.num_experts, self.num_experts_per_tok, self.norm_topk_prob,
                                 self.moe_intermediate_size, self.shared_expert_intermediate_size, p + "mlp.",
                                 names=MOE_NAMES)
            else:
                ffn = DenseFfnSpec(self.hidden_size, self.intermediate_size, p + "mlp.", names=MLP_NAMES)
            blocks.append(BlockSpec(
                mixer, ffn,
                NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, p + "post_attention_layernorm.weight")))
        return ModelPlan(
            architecture=ARCHITECTURE, hidden=self.hidden_size, vocab=self.vocab_size,
            max_positions=self.max_position_embeddings, blocks=blocks,
            schedule=[ScheduleEntry(i) for i in range(self.num_hidden_layers)],
            final_norm=NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
            embed_weight="model.embed_tokens.weight",
            head_weight=None if self.tie_word_embeddings else "lm_head.weight",
            stop_token_ids=self.stop_token_ids(),
            tolerated_suffixes=(".rotary_emb.inv_freq",),   # loader.rs:253-255
            # a tied checkpoint may still store the head; it is used if present (loader.rs:441-449)
            tied_head_name="lm_head.weight",
        )


# the checkpoint's tensor names below "model.layers.{i}." (loader.rs:87-91, :212-245, :512-556)
ATTENTION_NAMES = AttentionNames(q="q_proj", k="k_proj", v="v_proj", o="o_proj", weight=".weight", bias=".bias")
MLP_NAMES = SwiGluNames(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
MOE_NAMES = MoeNames(router="gate.weight", shared_gate="shared_expert_gate.weight", shared="shared_expert.",
                     expert="experts.{e}.", mlp=MLP_NAMES)

register_architecture(ARCHITECTURE, MODEL_TYPE, Qwen2MoeConfig)
