"""Binding a checkpoint's tensors to a model's parameters by name.

The rules follow the reference's loader
(crates/esp/src/infer/decoder/loader.rs:277-308, :425-462, :490-570): every
tensor the configuration calls for must be present with its exact shape, and a
checkpoint that carries a tensor nothing reads is refused (its weights would
compute something this decoder does not), except names that are known to be
derivable from the configuration.  All problems are gathered into one error.
"""
from __future__ import annotations

import torch

from ..errors import InvalidWeights
from .safetensors_io import open_model_folder, read_tensor

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


class FolderSource:
    """Tensors of a model folder (model.safetensors or its shards)."""

    def __init__(self, folder):
        self.metas = open_model_folder(folder)

    def names(self):
        return list(self.metas)

    def dtype(self, name):
        return self.metas[name].dtype

    def shape(self, name):
        return tuple(self.metas[name].shape)

    def read_into(self, name, view: torch.Tensor) -> None:
        t = read_tensor(self.metas[name])
        # non-finite weights are refused (crates/esp/src/infer/decoder/weight_format.rs:129-131)
        if not bool(torch.isfinite(t if t.dtype == torch.float32 else t.float()).all()):
            raise InvalidWeights(f"{name} holds values that are not finite")
        view.copy_(t.to(view.dtype) if t.dtype != view.dtype else t, non_blocking=False)


def check_names_and_shapes(specs: list, source, tolerated_suffixes=()) -> None:
    """One InvalidWeights that lists missing and unexpected tensors, wrong
    shapes and wrong dtypes; nothing if all is well."""
    wanted = {}
    for s in specs:
        if s.name in wanted and wanted[s.name].shape != s.shape:
            raise InvalidWeights(f"two parts declare {s.name} with different shapes")
        wanted[s.name] = s
    have = set(source.names())
    missing = sorted(n for n, s in wanted.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in wanted and not any(n.endswith(t) for t in tolerated_suffixes))
    wrong_shape, wrong_dtype = [], []
    for n in sorted(have & set(wanted)):
        if tuple(source.shape(n)) != tuple(wanted[n].shape):
            wrong_shape.append(f"{n}: stored {list(source.shape(n))}, expected {list(wanted[n].shape)}")
        if source.dtype(n) not in _FLOAT_DTYPES:
            wrong_dtype.append(f"{n}: stored as {source.dtype(n)}")
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = ["the checkpoint does not match the configuration:"]

    def add(title, items):
        if items:
            shown = items[:12]
            lines.append(f"  {title} ({len(items)}): " + "; ".join(shown) + (" ..." if len(items) > len(shown) else ""))

    add("missing tensors", missing)
    add("unexpected tensors (nothing in this configuration reads them)", unexpected)
    add("wrong shapes", wrong_shape)
    add("dtypes that are not floating point", wrong_dtype)
    raise InvalidWeights("\n".join(lines))


def load_into(root, source, rt, tolerated_suffixes=None) -> None:
    """Checks the source against the parameters of ``root`` (a model, or any
    part with its children), lets every part allocate its storage and fills it."""
    from ..parts import walk
    parts = list(walk(root))
    specs = [s for part in parts for s in part.param_specs()]
    if tolerated_suffixes is None:
        tolerated_suffixes = getattr(getattr(root, "plan", None), "tolerated_suffixes", ())
    check_names_and_shapes(specs, source, tolerated_suffixes)
    have = set(source.names())
    stored = {s.name: source.dtype(s.name) for s in specs if s.name in have}
    views = {}
    for part in parts:
        views.update(part.allocate(stored, rt))
    for name, view in views.items():
        if name not in have:
            raise InvalidWeights(f"a part asked for {name}, which the checkpoint lacks")
        source.read_into(name, view)
    for part in parts:
        part.finalize()
