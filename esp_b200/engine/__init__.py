from .engine import Engine, StepEntry, parse_dtype
from .model import DecoderModel

__all__ = ["Engine", "StepEntry", "parse_dtype", "DecoderModel"]
