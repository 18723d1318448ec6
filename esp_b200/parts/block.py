"""How the parts of one layer are arranged."""
from __future__ import annotations

import torch

from .base import Part, build, plain_delta, register


class PreNormResidualBlock(Part):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (crates/esp/src/infer/decoder/layer.rs:115-153).  The residual adds are
    folded into the norm that follows them: a part's output travels as
    ``pending`` until the next norm adds it to the 32-bit residual stream."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = build("norm", spec.mixer_norm, rt)
        self.mixer = build("mixer", spec.mixer, rt)
        self.ffn_norm = build("norm", spec.ffn_norm, rt)
        self.ffn = build("ffn", spec.ffn, rt)

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, x, pending, ctx, layer):
        rt = self.rt
        h = rt.ws.get("block_h", tuple(x.shape), rt.dtype)
        self.mixer_norm.forward(x, plain_delta(self.mixer_norm, pending), h)
        delta = self.mixer.forward(h, ctx, layer)
        h32 = None
        if rt.dtype != torch.float32 and getattr(self.ffn, "wants_f32_input", False):
            h32 = rt.ws.get("block_h32", tuple(x.shape), torch.float32)
        self.ffn_norm.forward(x, plain_delta(self.ffn_norm, delta), h, h32=h32)
        return self.ffn.forward(h, ctx, h32=h32)


register("block", "prenorm_residual", PreNormResidualBlock)
