"""Random weights from a configuration and a seed.

Every element is ``mean + std * z`` with z a standard normal drawn by a
counter-based generator: z depends on (seed, tensor name, flat index) only, so
a tensor's values do not depend on the order or the chunks in which tensors
are made.  The same integer stream drives a numpy version (used to write model
folders, needs no GPU) and a device kernel (used to fill a large model in
place); the two agree up to the last bit of the logarithm and cosine.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..errors import InvalidConfig
from .safetensors_io import write_safetensors

_M = (1 << 64) - 1


@dataclass(frozen=True)
class InitSpec:
    """Standard deviations: matrices N(0, weight_std); biases N(0, bias_std)
    (0: zeros); norm scales 1 + N(0, norm_std).  ``roles`` gives (mean, std)
    for any further role that a part's parameters may carry."""
    weight_std: float = 0.02
    bias_std: float = 0.0
    norm_std: float = 0.0
    roles: tuple = ()          # ((role, mean, std), ...)

    def mean_std(self, role: str):
        for name, mean, std in self.roles:
            if name == role:
                return float(mean), float(std)
        if role == "matrix":
            return 0.0, self.weight_std
        if role == "bias":
            return 0.0, self.bias_std
        if role == "norm_scale":
            return 1.0, self.norm_std
        raise InvalidConfig(f"no initialisation rule for parameter role {role!r}; give one in InitSpec.roles")


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M
    return _mix64((seed & _M) ^ h)


def _mix64_np(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def normal_values(key: int, count: int, mean: float, std: float) -> np.ndarray:
    """float32 [count]: the host version of the device fill."""
    out = np.empty(count, dtype=np.float32)
    chunk = 1 << 22
    for lo in range(0, count, chunk):
        hi = min(count, lo + chunk)
        with np.errstate(over="ignore"):
            i = np.arange(lo, hi, dtype=np.uint64) * np.uint64(2) + np.uint64(key)
            a = _mix64_np(i)
            b = _mix64_np(i + np.uint64(1))
        u1 = ((a >> np.uint64(40)).astype(np.float32) + np.float32(1.0)) * np.float32(1.0 / 16777216.0)
        u2 = (b >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
        z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(6.283185307179586) * u2)
        out[lo:hi] = np.float32(mean) + np.float32(std) * z.astype(np.float32)
    return out


class RandomSource:
    """Looks like a checkpoint to the loader; makes each tensor when asked.  A
    destination on the GPU is filled in place by the device kernel."""

    def __init__(self, specs: list, seed: int, init: InitSpec, dtype: torch.dtype):
        self.specs = {s.name: s for s in specs if not s.optional}
        self.seed = seed
        self.init = init
        self._dtype = dtype

    def names(self):
        return list(self.specs)

    def dtype(self, name):
        return self._dtype

    def shape(self, name):
        return tuple(self.specs[name].shape)

    def host_tensor(self, name) -> torch.Tensor:
        s = self.specs[name]
        mean, std = self.init.mean_std(s.role)
        count = int(np.prod(s.shape)) if s.shape else 1
        vals = normal_values(tensor_key(self.seed, name), count, mean, std) if std > 0 else np.full(
            count, mean, dtype=np.float32)
        return torch.from_numpy(vals).reshape(s.shape).to(self._dtype)

    def read_into(self, name, view: torch.Tensor) -> None:
        s = self.specs[name]
        mean, std = self.init.mean_std(s.role)
        if view.is_cuda and view.is_contiguous() and view.dtype in (torch.float32, torch.bfloat16) and std > 0:
            from ..csrc import ops
            if view.dtype == self._dtype or self._dtype == torch.float32:
                ops.normal_fill(view, tensor_key(self.seed, name), mean, std)
                return
            # stored narrower than kept: round through the stored dtype as a file would
            tmp = torch.empty(view.shape, dtype=self._dtype, device=view.device)
            ops.normal_fill(tmp, tensor_key(self.seed, name), mean, std)
            view.copy_(tmp)
            return
        view.copy_(self.host_tensor(name).to(view.dtype))


def parameter_specs(config) -> list:
    """Every tensor a model of this configuration reads (needs no GPU)."""
    from ..engine.model import DecoderModel
    from ..parts import Runtime
    model = DecoderModel(config.plan(), Runtime(None, torch.float32))
    return [s for part in model.all_parts() for s in part.param_specs()]


def write_model_folder(config, seed: int, folder, dtype: str = "bfloat16", init: InitSpec = InitSpec()) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` of a randomly
    initialised model.  ``dtype``: how the tensors are stored."""
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(dtype)
    if torch_dtype is None:
        raise InvalidConfig(f"dtype must be bfloat16 or float32, got {dtype!r}")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    src = RandomSource(parameter_specs(config), seed, init, torch_dtype)
    write_safetensors(folder / "model.safetensors", {n: src.host_tensor(n) for n in src.names()})
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    return folder
