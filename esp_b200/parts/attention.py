"""Softmax attention over the paged cache with grouped query heads."""
from __future__ import annotations

import numpy as np
import torch

from ..cache import KvLayout
from ..cache.book import PAGE
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

    graph_safe = True

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
    def _name(self, which: str, bias: bool = False) -> str:
        n = self.spec.names
        return self.spec.prefix + getattr(n, which) + (n.bias if bias else n.weight)

    def param_specs(self):
        s = self.spec
        specs = [ParamSpec(self._name("q"), (self.q_width, s.hidden), "matrix"),
                 ParamSpec(self._name("k"), (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(self._name("v"), (self.kv_width, s.hidden), "matrix"),
                 ParamSpec(self._name("o"), (s.hidden, self.q_width), "matrix")]
        if s.qkv_bias:
            specs += [ParamSpec(self._name("q", True), (self.q_width,), "bias"),
                      ParamSpec(self._name("k", True), (self.kv_width,), "bias"),
                      ParamSpec(self._name("v", True), (self.kv_width,), "bias")]
        if s.out_bias:
            specs.append(ParamSpec(self._name("o", True), (s.hidden,), "bias"))
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        names = [self._name("q"), self._name("k"), self._name("v")]
        dt = rt.matrix_dtype([stored[n] for n in names])
        self.w_qkv = torch.empty((self.qkv_width, s.hidden), dtype=dt, device=rt.device)
        self.w_o = torch.empty((s.hidden, self.q_width), dtype=rt.matrix_dtype([stored[self._name("o")]]),
                               device=rt.device)
        a, b = self.q_width, self.q_width + self.kv_width
        views = {names[0]: self.w_qkv[:a], names[1]: self.w_qkv[a:b], names[2]: self.w_qkv[b:],
                 self._name("o"): self.w_o}
        if s.qkv_bias:
            self.b_qkv = torch.empty(self.qkv_width, dtype=torch.float32, device=rt.device)
            views.update({self._name("q", True): self.b_qkv[:a], self._name("k", True): self.b_qkv[a:b],
                          self._name("v", True): self.b_qkv[b:]})
        if s.out_bias:
            self.b_o = torch.empty(s.hidden, dtype=torch.float32, device=rt.device)
            views[self._name("o", True)] = self.b_o
        return views

    # -- which kernel a step of n token rows gets, and the index lists it needs ----------
    def kernel_for(self, n: int, page: int = PAGE) -> str:
        s, rt = self.spec, self.rt
        if rt.dtype == torch.bfloat16:
            if s.head_dim in (64, 128, 192, 256) and n <= DECODE_ROWS and page == PAGE:
                return "split"         # few rows: split the keys over blocks so that the cache streams at full width
            if ops.attn_prefill_tc05_fits(s.head_dim, page):
                return "tc05"          # many rows, head size 64 or 128: scores and weighted values in tensor memory
            if s.head_dim <= 128 and page == 64:
                return "flash"
        return "plain"

    def step_arrays_key(self):
        return ("attention", self.rt.dtype, self.spec.head_dim)

    def step_arrays(self, step):
        """Tiles of new tokens for the two prefill kernels: (sequence, first new token) per tile; for the
        tensor-memory kernel the tiles that see the most keys come first (its blocks take them in order)."""
        kind = self.kernel_for(step.n_tokens)
        if kind == "tc05":
            rows = ops.ATTN_TC05_TILE_ROWS
            tiles = sorted(((i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)),
                           key=lambda sf: -(step.pasts[sf[0]] + min(sf[1] + rows, step.news[sf[0]])))
        elif kind == "flash":
            rows = 64
            tiles = [(i, f) for i, t in enumerate(step.news) for f in range(0, t, rows)]
        else:
            return {}
        return {f"attention.tiles{rows}.seq": np.asarray([t[0] for t in tiles], dtype=np.int32),
                f"attention.tiles{rows}.first": np.asarray([t[1] for t in tiles], dtype=np.int32)}

    # -- what it keeps per sequence ------------------------------------------------
    def kv_layout(self):
        return KvLayout(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def state_spec(self):
        return None

    # -- running ---------------------------------------------------------------
    def forward(self, h, ctx, layer):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        q = rt.ws.get("attn_q", (n, self.q_width), rt.dtype)
        fused = getattr(self.position, "project_rotate_store", None)
        if fused is None or not fused(h, self.w_qkv, self.b_qkv, ctx, q, layer, s.num_heads, s.num_kv_heads, s.head_dim,
                                      rt.status):
            qkv = rt.ws.get("attn_qkv", (n, self.qkv_width), torch.float32)
            linear(rt, h, self.w_qkv, qkv)
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
        kind = self.kernel_for(n, layer.page)
        if kind in ("tc05", "flash"):
            rows = ops.ATTN_TC05_TILE_ROWS if kind == "tc05" else 64
            tile_seq, tile_first = ctx.arrays.get(f"attention.tiles{rows}.seq"), ctx.arrays.get(f"attention.tiles{rows}.first")
            if tile_seq is None:
                kind = "plain"         # a step made without this part's lists (a caller that built its own context)
        if kind == "split":
            positions = table.shape[1] * layer.page
            group = s.num_heads // s.num_kv_heads
            kv_blocks = s.num_kv_heads * ((group + 15) // 16)
            # a windowed layer reads at most window + a page of each row, wherever in the table that lies
            span = min(positions, s.window + layer.page) if s.window else positions
            split = ops.attn_decode_split(n, kv_blocks, span, s.head_dim, rt.sm_count)
            n_splits = (positions + split - 1) // split
            part_o = rt.ws.get("attn_part_o", (n, s.num_heads, n_splits, s.head_dim), torch.float32)
            part_ml = rt.ws.get("attn_part_ml", (n, s.num_heads, n_splits, 2), torch.float32)
            if getattr(rt, "attn_counters", None) is None:
                rt.attn_counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=rt.device)
            ops.attn_decode(q, layer.k, layer.v, o, part_o, part_ml, rt.attn_counters, ctx.tok_seq, ctx.tok_pos, table, layer.page,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.window, split, n_splits, rt.status,
                            seq_past=ctx.seq_past if layer.writes else None)
        elif kind == "tc05":
            ops.attn_prefill_tc05(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past,
                                  table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
        elif kind == "flash":
            ops.attn_prefill(q, layer.k, layer.v, o, tile_seq, tile_first, ctx.seq_start, ctx.seq_past,
                             table, layer.page, s.num_heads, s.num_kv_heads, s.head_dim, s.window, rt.status)
        else:
            ops.attn_simt(q, layer.k, layer.v, o, ctx.tok_seq, ctx.tok_pos, table, layer.page, s.num_heads,
                          s.num_kv_heads, s.head_dim, s.window, rt.status)


register("mixer", "attention", Attention)
