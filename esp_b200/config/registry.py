"""One registry from an architecture's name to its typed configuration.

Lookup follows the reference (crates/esp/src/infer/decoder/config.rs:25-34,
:397-419): ``architectures[0]`` decides, ``model_type`` is the fallback, and
when both are present they must agree.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Union

from ..errors import InvalidConfig, Unsupported

_BY_ARCHITECTURE: dict = {}
_BY_MODEL_TYPE: dict = {}


def register_architecture(architecture: str, model_type: str, config_cls) -> None:
    """``config_cls`` needs ``from_dict(dict) -> config`` and the config needs
    ``plan() -> ModelPlan`` and ``to_dict()``."""
    _BY_ARCHITECTURE[architecture] = (model_type, config_cls)
    _BY_MODEL_TYPE[model_type] = (architecture, config_cls)


def supported_architectures() -> list:
    return sorted(_BY_ARCHITECTURE)


def config_from_dict(raw: dict):
    if not isinstance(raw, dict):
        raise InvalidConfig("config.json must hold a JSON object")
    if raw.get("text_config") is not None:
        raise Unsupported("text_config", "multimodal configs nest the language model; only a flat decoder config runs")
    archs = raw.get("architectures")
    model_type = raw.get("model_type")
    if archs is not None and (not isinstance(archs, list) or not all(isinstance(a, str) for a in archs)):
        raise InvalidConfig("architectures must be a list of strings")
    if model_type is not None and model_type not in _BY_MODEL_TYPE:
        raise Unsupported("model_type", f"{model_type!r}; supported: {sorted(_BY_MODEL_TYPE)}")
    for a in archs or []:
        if a not in _BY_ARCHITECTURE:
            raise Unsupported("architectures", f"{a!r}; supported: {supported_architectures()}")
    if archs:
        want_type, cls = _BY_ARCHITECTURE[archs[0]]
        if model_type is not None and model_type != want_type:
            raise InvalidConfig(f"architectures {archs[0]!r} and model_type {model_type!r} disagree")
    elif model_type is not None:
        _, cls = _BY_MODEL_TYPE[model_type]
    else:
        raise InvalidConfig("config.json names neither architectures nor model_type")
    return cls.from_dict(raw)


def config_from_json(source: Union[str, bytes, Path]):
    """``source``: a path to config.json (or to the model folder) or its bytes."""
    if isinstance(source, (bytes, bytearray)):
        text = bytes(source).decode("utf-8")
    else:
        p = Path(source)
        if p.is_dir():
            p = p / "config.json"
        if not p.is_file():
            raise InvalidConfig(f"no config.json at {p}")
        text = p.read_text()
    try:
        raw = json.loads(text)
    except json.JSONDecodeError as e:
        raise InvalidConfig(f"config.json is not valid JSON: {e}") from None
    return config_from_dict(raw)
