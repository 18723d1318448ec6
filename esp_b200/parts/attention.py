"""Softmax attention over the paged cache with grouped query heads."""
from __future__ import annotations

import torch

from ..cache import KvLayout
from ..csrc import ops
from ..errors import Unsupported
from .base import ParamSpec, Part, build, register
from .linear import linear
from .position import NoPosition


DECODE_ROWS = 128      # steps with at most this many token rows use the split-key kernel


class Attention(Part):
    """q/k/v projection (+bias), position encoding of q and k, cache write,
    causal (optionally windowed) softmax attention, output projection
    (crates/esp/src/infer/decoder/attention.rs:292-404).  Query head i reads
    key/value head i // (num_heads / num_kv_heads)."""

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        s = spec
        if s.head_dim % 8 != 0 or s.head_dim > 256:
            raise Unsupported("head_dim", f"{s.head_dim}; the attention kernels take head sizes that are multiples "
                                          f"of 8 up to 256")
        if s.num_heads % s.num_kv_heads != 0:
            raise Unsupported("num_key_value_heads", f"{s.num_kv_heads} does not divide {s.num_heads} heads")
        self.q_width = s.num_heads * s.head_dim
        self.kv_width = s.num_kv_heads * s.head_dim
        self.qkv_width = self.q_width + 2 * self.kv_width
        # layers with the same encoding share one part (and its tables)
        key = ("position", s.position)
        if key not in rt.shared_parts:
            rt.shared_parts[key] = build("position", s.position, rt) if s.position is not None else NoPosition(None, rt)
        self.position = rt.shared_parts[key]
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def children(self):
        return [self.position]

    # -- parameters ----------------------------------------------------------
    def param_specs(self):
        s, p = self.spec, self.spec.prefix
        specs = [ParamSpec(p + "q_proj.weight", (self.q_width, s.hidden), "matrix"),
                 ParamSpec(p + "k_proj.weight", (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(p + "v_proj.weight", (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(p + "o_proj.weight", (s.hidden, self.q_width), "matrix")]
        if s.qkv_bias:
            specs += [ParamSpec(p + "q_proj.bias", (self.q_width,), "bias"),
                      ParamSpec(p + "k_proj.bias", (self.kv_width,), "bias"),
                      ParamSpec(p + "v_proj.bias", (self.kv_width,), "bias")]
        if s.out_bias:
            specs.append(ParamSpec(p + "o_proj.bias", (s.hidden,), "bias"))
        return specs

    def allocate(self, stored, rt):
        s, p = self.spec, self.spec.prefix
        names = [p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"]
        dt = rt.matrix_dtype([stored[n] for n in names])
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=dt, device=rt.device)
        self.w_o = torch.empty((s.hidden, self.q_width), dtype=rt.matrix_dtype([stored[p + "o_proj.weight"]]),
                               device=rt.device)
        a, b = self.q_width, self.q_width + self.kv_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:],
                 p + "o_proj.weight": self.w_o}
        if s.qkv_bias:
            self.b_qkv = torch.empty(self.qkv_width, dtype=torch.float32, device=rt.device)
            views.update({p + "q_proj.bias": self.b_qkv[:a], p + "k_proj.bias": self.b_qkv[a:b],
                          p + "v_proj.bias": self.b_qkv[b:]})
        if s.out_bias:
            self.b_o = torch.empty(s.hidden, dtype=torch.float32, device=rt.device)
            views[p + "o_proj.bias"] = self.b_o
        return views

    # -- what it keeps per sequence ------------------------------------------------
    def kv_layout(self):
        return KvLayout(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def state_spec(self):
        return None

    # -- running ---------------------------------------------------------------
    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
        linear(rt, h, self.w_qkv, qkv)
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        self.position.rotate_and_store(qkv, self.b_qkv, ctx, q, layer, s.num_heads, s.num_kv_heads, s.head_dim,
                                       rt.status)
        o = rt.ws.get("attn_o", (n, self.q_width), rt.dtype)
        self.attend(q, o, ctx, layer)
        y = rt.ws.get("mixer_out", (n, s.hidden), torch.float32)
        linear(rt, o, self.w_o, y)
        if self.b_o is not None:
            y.add_(self.b_o)
        return y

    def attend(self, q, o, ctx, layer):
        s, rt = self.spec, self.rt
        table = ctx.block_tables[layer.group]
        n = q.shape[0]
        if rt.dtype == torch.bfloat16 and s.head_dim in (64, 128, 192, 256) and n <= DECODE_ROWS:
            # few rows: split the keys over blocks so that the cache streams at full width
            positions = table.shape[1] * layer.page
            group = s.num_heads // s.num_kv_heads
            kv_blocks = s.num_kv_heads * ((group + 15) // 16)
            split = ops.attn_decode_split(n, kv_blocks, positions)
            n_splits = (positions + split - 1) // split
            part_o = rt.ws.get("attn_part_o", (n, s.num_heads, n_splits, s.head_dim), torch.float32)
            part_ml = rt.ws.get("attn_part_ml", (n, s.num_heads, n_splits, 2), torch.float32)
            if getattr(rt, "attn_counters", None) is None:
                rt.attn_counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=rt.device)
            ops.attn_decode(q, layer.k, layer.v, o, part_o, part_ml, rt.attn_counters, ctx.tok_seq, ctx.tok_pos, table, layer.page,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.window, split, n_splits, rt.status)
            return
        if rt.dtype == torch.bfloat16 and ops.attn_prefill_tc05_fits(s.head_dim, layer.page) and ctx.q_wide_seq is not None:
            # many rows, head size 64 or 128: scores and weighted values in tensor memory (tcgen05)
            ops.attn_prefill_tc05(q, layer.k, layer.v, o, ctx.q_wide_seq, ctx.q_wide_first, ctx.seq_start, ctx.seq_past,
                                  table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
            return
        if rt.dtype == torch.bfloat16 and s.head_dim <= 128 and layer.page == 64:
            ops.attn_prefill(q, layer.k, layer.v, o, ctx.q_tile_seq, ctx.q_tile_first, ctx.seq_start, ctx.seq_past,
                             table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
            return
        ops.attn_simt(q, layer.k, layer.v, o, ctx.tok_seq, ctx.tok_pos, table, layer.page, s.num_heads,
                      s.num_kv_heads, s.head_dim, s.window, rt.status)


register("mixer", "attention", Attention)
