"""Feed-forward parts: a dense SwiGLU MLP and the sparse block with routed
experts and a gated shared expert."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamSpec, Part, register
from .linear import grouped_linear, grouped_swiglu_linear, grouped_uses_tc05, linear, swiglu_linear


class DeferredMoeCombine:
    """What a sparse block hands on instead of its output when nothing has to see that output by itself:
    the pieces of the combine.  A norm that knows the fused kernel adds and normalises in one launch
    (``fused_add_rmsnorm``); anything else calls ``materialize()`` and gets the plain tensor."""

    def __init__(self, rt, expert_out, ids, inverse, gate, shared, width):
        self.rt, self.expert_out, self.ids, self.inverse, self.gate, self.shared = rt, expert_out, ids, inverse, gate, shared
        self.width = width

    def materialize(self):
        y = self.rt.ws.get("ffn_out", (self.ids.shape[0], self.width), torch.float32)
        ops.moe_combine(self.expert_out, self.ids, self.inverse, self.gate, self.shared, y)
        return y

    def fused_add_rmsnorm(self, x, gamma, h, eps, rows, write_x, h32):
        ops.moe_combine_add_rmsnorm(self.expert_out, self.ids, self.inverse, self.gate, self.shared, x, gamma, h, eps,
                                    rows=rows, write_x=write_x, h32=h32)


# Steps with at least AHEAD_ROWS rows start the shared expert's first product on a second stream before the
# router, on all SMs but ROUTING_SMS: the router and the permutation are a chain of short launches that leaves
# the device idle, and they find room on the SMs left over (2,048 tokens, 24 layers: 12.7 -> 12.2 ms; with 4 or 16
# SMs left over 12.6 and 12.5 ms).  Below about 768 rows it does not pay (one prompt of 400 tokens: 7.4 -> 7.7 ms;
# 768: even; 1,024: 8.9 -> 8.3 ms).
AHEAD_ROWS = 768
EARLY_SECOND_PRODUCT_ROWS = 16
ROUTING_SMS = 8
SIDE_STREAM_ROWS = 64      # steps with at most this many rows run the shared expert on a second stream


def _swiglu_mlp(rt, h, w_gate_up, w_down, out, tag):
    """out = down(silu(gate h) * (up h)); w_gate_up is [2I, H], gate rows first."""
    n = h.shape[0]
    inter = w_gate_up.shape[0] // 2
    act = rt.ws.get(tag + "_act", (n, inter), rt.dtype)
    swiglu_linear(rt, h, w_gate_up, act, tag)
    linear(rt, act, w_down, out)
    return out


class DenseSwiGlu(Part):
    """y = W_d(silu(W_g h) * (W_u h)), no biases
    (crates/esp/src/infer/decoder/moe.rs:87-89, :143-148)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        return [ParamSpec(p + n.gate, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.up, (s.intermediate, s.hidden), "matrix"),
                ParamSpec(p + n.down, (s.hidden, s.intermediate), "matrix")]

    def allocate(self, stored, rt):
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        dt = rt.matrix_dtype([stored[p + n.gate], stored[p + n.up]])
        self.w_gate_up = torch.empty((2 * s.intermediate, s.hidden), dtype=dt, device=rt.device)
        self.w_down = torch.empty((s.hidden, s.intermediate), dtype=rt.matrix_dtype([stored[p + n.down]]),
                                  device=rt.device)
        return {p + n.gate: self.w_gate_up[:s.intermediate], p + n.up: self.w_gate_up[s.intermediate:],
                p + n.down: self.w_down}

    def forward(self, h, ctx, h32=None):
        rt = self.rt
        n = h.shape[0]
        y = rt.ws.get("ffn_out", (n, self.spec.hidden), torch.float32)
        step = rt.ffn_chunk_tokens
        for a in range(0, n, step):
            b = min(n, a + step)
            _swiglu_mlp(rt, h[a:b], self.w_gate_up, self.w_down, y[a:b], "dense")
        return y


class MoeSwiGluShared(Part):
    """Router (32-bit softmax over all experts, top-k, ties to the lower id,
    optional renormalisation), routed SwiGLU experts whose outputs are scaled
    by their routing weight and summed in ascending expert id, plus a shared
    SwiGLU expert scaled by sigmoid(h . w_shared_gate)
    (crates/esp/src/infer/decoder/moe.rs:135-256)."""

    graph_safe = True

    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt
        self.w_router = self.w_shared_gate = None
        self.w_gate_up = self.w_down = None            # [E, 2Im, H], [E, H, Im]
        self.w_shared_gate_up = self.w_shared_down = None
        # experts with at least one token, summed over this block's calls (a device counter; nothing waits for it)
        self.expert_reads = rt.new_counter("expert_reads")

    def _names(self):
        """(router, shared gate, shared (gate, up, down), [per expert (gate, up, down)])"""
        s, p, n = self.spec, self.spec.prefix, self.spec.names
        mlp = lambda q: (q + n.mlp.gate, q + n.mlp.up, q + n.mlp.down)
        return (p + n.router, p + n.shared_gate, mlp(p + n.shared),
                [mlp(p + n.expert.format(e=e)) for e in range(s.num_experts)])

    def param_specs(self):
        s = self.spec
        router, shared_gate, shared, experts = self._names()
        specs = [ParamSpec(router, (s.num_experts, s.hidden), "matrix"),
                 ParamSpec(shared_gate, (1, s.hidden), "matrix"),
                 ParamSpec(shared[0], (s.shared_intermediate, s.hidden), "matrix"),
                 ParamSpec(shared[1], (s.shared_intermediate, s.hidden), "matrix"),
                 ParamSpec(shared[2], (s.hidden, s.shared_intermediate), "matrix")]
        for gate, up, down in experts:
            specs += [ParamSpec(gate, (s.expert_intermediate, s.hidden), "matrix"),
                      ParamSpec(up, (s.expert_intermediate, s.hidden), "matrix"),
                      ParamSpec(down, (s.hidden, s.expert_intermediate), "matrix")]
        return specs

    def allocate(self, stored, rt):
        s = self.spec
        dev = rt.device
        E, Im, Is, H = s.num_experts, s.expert_intermediate, s.shared_intermediate, s.hidden
        router, shared_gate, shared, experts = self._names()
        rdt = rt.matrix_dtype([stored[router], stored[shared_gate]])
        self.w_router = torch.empty((E, H), dtype=rdt, device=dev)
        self.w_shared_gate = torch.empty((1, H), dtype=rdt, device=dev)
        gu_dt = rt.matrix_dtype([stored[n] for g, u, _d in experts for n in (g, u)])
        self.w_gate_up = torch.empty((E, 2 * Im, H), dtype=gu_dt, device=dev)
        self.w_down = torch.empty((E, H, Im), dtype=rt.matrix_dtype([stored[d] for _g, _u, d in experts]), device=dev)
        sdt = rt.matrix_dtype([stored[shared[0]], stored[shared[1]]])
        self.w_shared_gate_up = torch.empty((2 * Is, H), dtype=sdt, device=dev)
        self.w_shared_down = torch.empty((H, Is), dtype=rt.matrix_dtype([stored[shared[2]]]), device=dev)
        views = {router: self.w_router, shared_gate: self.w_shared_gate,
                 shared[0]: self.w_shared_gate_up[:Is], shared[1]: self.w_shared_gate_up[Is:],
                 shared[2]: self.w_shared_down}
        for e, (gate, up, down) in enumerate(experts):
            views[gate] = self.w_gate_up[e, :Im]
            views[up] = self.w_gate_up[e, Im:]
            views[down] = self.w_down[e]
        return views

    wants_f32_input = True      # the router works from unrounded rows

    def forward(self, h, ctx, h32=None):
        rt = self.rt
        n = h.shape[0]
        step = rt.ffn_chunk_tokens
        if n <= step and self.spec.hidden % 4 == 0 and self.spec.hidden <= 16384:
            # one chunk: leave the combine to the norm that follows (one launch for combine, add and norm)
            return self._forward_rows(h, None, ctx, 0, h32 if h32 is not None else h)
        y = rt.ws.get("ffn_out", (n, self.spec.hidden), torch.float32)
        for a in range(0, n, step):
            b = min(n, a + step)
            self._forward_rows(h[a:b], y[a:b], ctx, a, h32[a:b] if h32 is not None else h[a:b])
        return y

    def _forward_rows(self, h, y, ctx, row0, router_in):
        s, rt = self.spec, self.rt
        n, k, E, Im, H = h.shape[0], s.top_k, s.num_experts, s.expert_intermediate, s.hidden
        ws = rt.ws
        ids = ws.get("moe_ids", (n, k), torch.int32)
        wts = ws.get("moe_w", (n, k), torch.float32)
        gate = ws.get("moe_gate", (n,), torch.float32)
        probs = None
        if rt.record_routing:
            probs = torch.empty((n, E), dtype=torch.float32, device=rt.device)
        offsets = ws.get("moe_offsets", (E + 1,), torch.int32)
        perm_token = ws.get("moe_perm_token", (n * k,), torch.int32)
        perm_weight = ws.get("moe_perm_weight", (n * k,), torch.float32)
        inverse = ws.get("moe_inverse", (n, k), torch.int32)
        tiles = None
        shared = ws.get("moe_shared_out", (n, H), torch.float32)
        beside = n <= SIDE_STREAM_ROWS and rt.side_stream is not None
        ahead = not beside and n >= AHEAD_ROWS and rt.side_stream is not None and rt.dtype == torch.bfloat16
        if ahead:
            main = torch.cuda.current_stream()
            rt.side_stream.wait_stream(main)
            act_s = ws.get("moe_shared_act", (n, s.shared_intermediate), rt.dtype)
            with torch.cuda.stream(rt.side_stream):
                swiglu_linear(rt, h, self.w_shared_gate_up, act_s, "moe_shared", max_ctas=max(2, rt.sm_count - ROUTING_SMS))
        if beside:
            # few rows: the shared expert depends neither on the router nor on the routing, so it runs beside
            # them and the routed experts on a second stream (in a captured step: a parallel branch of the graph)
            main = torch.cuda.current_stream()
            rt.side_stream.wait_stream(main)
            with torch.cuda.stream(rt.side_stream):
                _swiglu_mlp(rt, h, self.w_shared_gate_up, self.w_shared_down, shared, "moe_shared")
        uses_tc05 = grouped_uses_tc05(h, self.w_gate_up, n * k, n) and Im % 8 == 0
        if uses_tc05:
            max_tiles = (n * k + ops.TC05_TILE_ROWS - 1) // ops.TC05_TILE_ROWS + E
            tiles = (ws.get("moe_tile_group", (max_tiles,), torch.int32),
                     ws.get("moe_tile_row0", (max_tiles,), torch.int32),
                     ws.get("moe_tile_count", (max_tiles,), torch.int32), ws.get("moe_n_tiles", (1,), torch.int32))
        if n <= ops.ROUTE_SMALL_TOKENS and ops.route_small_fits(H, E):
            # few tokens: router and permutation (and the tile list, when the tensor-core products follow) in two
            # short launches
            logits = ws.get("moe_logits", (n, E + 1), torch.float32)
            ops.route_small(router_in, self.w_router, self.w_shared_gate, logits, ids, wts, gate, k, s.norm_topk,
                            offsets, perm_token, perm_weight, inverse, rt.status, probs, distinct=self.expert_reads,
                            tiles=tiles)
        else:
            ops.router_topk(router_in, self.w_router, self.w_shared_gate, ids, wts, gate, k, s.norm_topk, rt.status,
                            probs, logits=ws.get("moe_logits", (n, E + 1), torch.float32))
            ops.moe_permute(ids, wts, E, offsets, perm_token, perm_weight, inverse, rt.status, tiles=tiles,
                            distinct=self.expert_reads)
        if rt.record_routing:
            ctx.aux.setdefault("routing", []).append((s.prefix, row0, ids.clone(), wts.clone(), probs))
        if ahead:
            main.wait_stream(rt.side_stream)
        expert_out = self.experts(h, offsets, perm_token, perm_weight, n * k, n, tiles)
        if beside:
            main.wait_stream(rt.side_stream)
        elif ahead:
            linear(rt, act_s, self.w_shared_down, shared)
        else:
            _swiglu_mlp(rt, h, self.w_shared_gate_up, self.w_shared_down, shared, "moe_shared")
        if y is None:
            return DeferredMoeCombine(rt, expert_out, ids, inverse, gate, shared, H)
        ops.moe_combine(expert_out, ids, inverse, gate, shared, y)
        return y

    def experts(self, h, offsets, perm_token, perm_weight, rows, max_rows, tiles=None):
        """expert_out[r] = weight[r] * down_e(silu(gate_e x) * (up_e x)) for every
        permuted row r, x = h[perm_token[r]], e the expert whose range holds r.
        ``max_rows``: no expert has more rows than this (a token names an expert once)."""
        s, rt = self.spec, self.rt
        act = rt.ws.get("moe_act", (rows, s.expert_intermediate), rt.dtype)
        grouped_swiglu_linear(rt, h, self.w_gate_up, act, offsets, perm_token, rows, max_rows, "moe", tiles)
        out = rt.ws.get("moe_expert_out", (rows, s.hidden), torch.float32)
        # the routing was complete before the first product started: the second may look its groups up and ask for
        # its weights while the first still runs.  Only for few rows, where the first product is one wave of
        # blocks and the second's blocks take no room from blocks yet to start (batch 1 +1.2 %, batch 4 +1.5 %,
        # batch 8 -0.3 %).
        grouped_linear(rt, act, self.w_down, out, offsets, perm_weight, rows, max_rows, tiles,
                       offsets_ready=rows <= EARLY_SECOND_PRODUCT_ROWS)
        return out


register("ffn", "swiglu", DenseSwiGlu)
register("ffn", "moe_swiglu_shared", MoeSwiGluShared)
