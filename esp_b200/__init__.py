"""esp_b200: a small, whole generation library for one GPU (sm_100a)."""
from .errors import (Backend, CacheFull, InferError, InvalidConfig, InvalidRequest, InvalidWeights, PromptTooLong,
                     Unsupported)

__all__ = ["Backend", "CacheFull", "InferError", "InvalidConfig", "InvalidRequest", "InvalidWeights", "PromptTooLong",
           "Unsupported", "load", "DecoderProvider", "GenerationRequest", "DecoderGeneration"]


def __getattr__(name):
    if name in ("load", "DecoderProvider", "GenerationRequest", "DecoderGeneration", "ModelCapability"):
        from . import provider
        return getattr(provider, name)
    raise AttributeError(name)
