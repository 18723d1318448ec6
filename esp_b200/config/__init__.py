from .plan import (AttentionSpec, BlockSpec, DenseFfnSpec, ModelPlan, MoeFfnSpec, NormSpec, PositionSpec,
                   ScheduleEntry)
from .registry import config_from_dict, config_from_json, register_architecture, supported_architectures
from .qwen2_moe import Qwen2MoeConfig

__all__ = ["AttentionSpec", "BlockSpec", "DenseFfnSpec", "ModelPlan", "MoeFfnSpec", "NormSpec", "PositionSpec",
           "ScheduleEntry", "config_from_dict", "config_from_json", "register_architecture",
           "supported_architectures", "Qwen2MoeConfig"]
