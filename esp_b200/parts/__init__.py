from .base import ParamSpec, Part, Runtime, StepContext, Workspace, build, register, walk
from . import attention, block, ffn, norm, position  # noqa: F401  (fills the registries)

__all__ = ["ParamSpec", "Part", "Runtime", "StepContext", "Workspace", "build", "register", "walk"]
