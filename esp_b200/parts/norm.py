"""RMSNorm fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamSpec, Part, register


class RmsNorm(Part):
    """h = (x + delta) * rsqrt(mean((x + delta)^2) + eps) * weight, in 32-bit
    (crates/esp/src/infer/decoder/layer.rs:27-33)."""

    graph_safe = True
    takes_deferred = True      # a deferred expert sum is added and normalised here in one launch

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.spec.weight, (self.spec.width,), "norm_scale")]

    def allocate(self, stored, rt):
        self.weight = torch.empty(self.spec.width, dtype=torch.float32, device=rt.device)
        return {self.spec.weight: self.weight}

    def forward(self, x, delta, h, rows=None, write_x=True, h32=None):
        if hasattr(delta, "fused_add_rmsnorm"):
            # the producer left its last step (an ordered sum) to be done here, in the same launch
            delta.fused_add_rmsnorm(x, self.weight, h, self.spec.eps, rows, write_x, h32)
            return h
        ops.add_rmsnorm(x, delta, self.weight, h, self.spec.eps, rows=rows, write_x=write_x, h32=h32)
        return h


register("norm", "rmsnorm", RmsNorm)
