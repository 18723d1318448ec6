"""The decoder as the engine runs it: an embedding, blocks called in the order
of the plan's schedule, a final norm and a head."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..parts import ParamSpec, Part, build, walk
from ..parts.base import plain_delta
from ..parts.linear import linear


class DecoderModel(Part):
    """Embedding (rows times ``plan.embed_scale``), the blocks in the order of
    the schedule, the final norm and the head on the wanted rows (with
    ``plan.logit_softcap`` if the plan has one)."""

    graph_safe = True

    def __init__(self, plan, rt):
        self.plan = plan
        self.rt = rt
        self.blocks = [build("block", spec, rt) for spec in plan.blocks]
        self.final_norm = build("norm", plan.final_norm, rt)
        self.embed = None
        self.head = None
        for i, e in enumerate(plan.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the plan has {len(self.blocks)}")

    def children(self):
        return [*self.blocks, self.final_norm]

    # -- parameters ---------------------------------------------------------------
    def param_specs(self):
        p = self.plan
        specs = [ParamSpec(p.embed_weight, (p.vocab, p.hidden), "matrix")]
        if p.head_weight is not None:
            specs.append(ParamSpec(p.head_weight, (p.vocab, p.hidden), "matrix"))
        elif p.tied_head_name is not None:
            # a tied model may still carry an explicit head; it is used if present
            specs.append(ParamSpec(p.tied_head_name, (p.vocab, p.hidden), "matrix", optional=True))
        return specs

    def allocate(self, stored, rt):
        p = self.plan
        self.embed = torch.empty((p.vocab, p.hidden), dtype=rt.matrix_dtype([stored[p.embed_weight]]), device=rt.device)
        views = {p.embed_weight: self.embed}
        head_name = p.head_weight or p.tied_head_name
        if head_name is not None and head_name in stored:
            self.head = torch.empty((p.vocab, p.hidden), dtype=rt.matrix_dtype([stored[head_name]]), device=rt.device)
            views[head_name] = self.head
        else:
            self.head = self.embed
        return views

    def all_parts(self):
        return list(walk(self))

    def cache_requests(self):
        """(KvLayout or None, StateSpec or None, cache_of) per schedule entry."""
        out = []
        for e in self.plan.schedule:
            mixer = self.blocks[e.layer].mixer
            layout = mixer.kv_layout() if hasattr(mixer, "kv_layout") else None
            state = mixer.state_spec() if hasattr(mixer, "state_spec") else None
            out.append((layout, state, e.cache_of))
        return out

    # -- running ------------------------------------------------------------------
    def forward(self, ctx, cache):
        """Logits [R, vocab] float32 at ctx.want_rows (R may be 0)."""
        rt, p = self.rt, self.plan
        n = ctx.n_tokens
        x = rt.ws.get("residual", (n, p.hidden), torch.float32)
        ops.embed_gather(self.embed, ctx.tok_ids, x, rt.status, scale=p.embed_scale)
        pending = None
        for idx, entry in enumerate(p.schedule):
            pending = self.blocks[entry.layer].forward(x, pending, ctx, cache.layers[idx])
        r = ctx.want_rows.shape[0]
        logits = torch.empty((r, p.vocab), dtype=torch.float32, device=rt.device)
        if r == 0:
            return logits
        h = rt.ws.get("head_in", (r, p.hidden), rt.dtype)
        self.final_norm.forward(x, plain_delta(self.final_norm, pending), h, rows=ctx.want_rows, write_x=False)
        linear(rt, h, self.head, logits)
        if p.logit_softcap is not None:
            ops.softcap(logits, p.logit_softcap)
        return logits
