"""Position encodings: they act on the new queries and keys between the
projection and the cache write."""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .base import Part, register


class RopeSplitHalf(Part):
    """Rotary encoding over the first ``rotary_dim`` columns of each head, pairs
    (i, i + rotary_dim/2).  Frequencies 1/theta^(2i/d) and angles p*f are taken
    in 32-bit on the host once (crates/esp/src/infer/decoder/attention.rs:58-95)
    and kept as cos/sin tables [max_positions, rotary_dim/2]."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.cos = self.sin = None

    def finalize(self):
        if self.cos is not None:
            return
        spec, rt = self.spec, self.rt
        half = spec.rotary_dim // 2
        i = np.arange(half, dtype=np.float32)
        freq = (np.float32(1.0) / np.power(np.float32(spec.theta), (np.float32(2.0) * i) / np.float32(spec.rotary_dim)))
        ang = np.arange(spec.max_positions, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(rt.device).contiguous()
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(rt.device).contiguous()

    def rotate_and_store(self, qkv, bias, ctx, q_out, layer, nh, nkv, hd, status):
        table = ctx.block_tables[layer.group] if layer.group is not None else None
        ops.rope_kvwrite(qkv, bias, ctx.tok_seq, ctx.tok_pos, self.cos, self.sin, self.spec.rotary_dim, q_out,
                         layer.k, layer.v, table, layer.page, nh, nkv, hd, layer.writes, status)

    def project_rotate_store(self, h, w_qkv, bias, ctx, q_out, layer, nh, nkv, hd, status) -> bool:
        """Optional short cut of a position part: the packed projection, this encoding and the cache write
        in one kernel.  False: not for these sizes; the caller projects and calls ``rotate_and_store``."""
        if (h.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or self.spec.rotary_dim != hd
                or layer.group is None or not ops.qkv_rope_skinny_fits(h.shape[0], h.shape[1], hd)):
            return False
        ops.qkv_rope_skinny(h, w_qkv, bias, ctx.tok_seq, ctx.tok_pos, self.cos, self.sin, q_out, layer.k, layer.v,
                            ctx.block_tables[layer.group], layer.page, nh, nkv, hd, layer.writes, status)
        return True


class NoPosition(Part):
    """No encoding: queries and keys are stored as projected."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec

    def rotate_and_store(self, qkv, bias, ctx, q_out, layer, nh, nkv, hd, status):
        table = ctx.block_tables[layer.group] if layer.group is not None else None
        ops.rope_kvwrite(qkv, bias, ctx.tok_seq, ctx.tok_pos, None, None, 0, q_out, layer.k, layer.v, table,
                         layer.page, nh, nkv, hd, layer.writes, status)


register("position", "rope_split_half", RopeSplitHalf)
register("position", "none", NoPosition)
