"""What every part of a layer has in common: its parameters, the registries
that map a spec's ``kind`` to a builder, and the runtime that parts run in.

A part never learns which model it is in.  It is built from its spec (sizes
and constants) and a ``Runtime``; it names its tensors, says where each one is
to be stored, and then runs on packed token rows.

Interfaces (all tensors live on the GPU; N = tokens of the step, H = width):

* norm:      ``forward(x, delta, h, rows=None, write_x=True, h32=None)``: x [N,H] float32 is the residual stream;
             ``delta`` (float32 [N,H], None, or a deferred output with ``materialize()``) is added to it first; h receives the normed rows in the
             activation dtype.
* mixer:     ``forward(h, ctx, layer) -> delta`` float32 [N,H]; ``kv_layout()`` and ``state_spec()`` say
             what it keeps per sequence (``layer`` is a ``cache.LayerCache``).
* ffn:       ``forward(h, ctx, h32=None) -> delta`` float32 [N,H]; a part with ``wants_f32_input = True``
             also gets the normed rows unrounded (float32) when the activation dtype is narrower.
* position:  ``rotate_and_store(qkv, bias, ctx, q_out, layer, nh, nkv, hd, status)``: encodes the new queries and
             keys (float32 in ``qkv``) and stores keys and values in the cache.  Optional:
             ``project_rotate_store(h, w_qkv, bias, ctx, q_out, layer, nh, nkv, hd, status) -> bool`` does the
             packed projection as well, in one kernel, where the part has one for the sizes at hand.
* block:     ``forward(x, pending, ctx, layer) -> pending``: runs its parts in its arrangement.

Per-step index lists.  A part that needs lists of its own on the device (tiles
of new tokens for an attention kernel, chunk boundaries for a scan) returns them
from ``step_arrays(step)`` as named int32 numpy arrays, made from the host-side
description of the step; the engine copies them to the device with the rest of
the step's metadata and hands them back as ``ctx.arrays[name]``.  The engine
itself knows none of these lists.

Captured steps.  A decode step is replayed from a CUDA graph only if every part
of the model has ``graph_safe = True``.  A graph-safe part does the same
launches with the same addresses for every step of the same shape (number of
sequences, page-table stride, sizes of its step arrays): it reads nothing from
``ctx.host`` while it runs, never syncs with the host, and takes slots,
positions and page tables from the device tensors of the context.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..errors import Backend, InvalidConfig


@dataclass(frozen=True)
class ParamSpec:
    name: str                 # tensor name in the checkpoint
    shape: tuple
    role: str                 # "matrix" | "bias" | "norm_scale"
    optional: bool = False


@dataclass(frozen=True)
class StepHost:
    """What a step is, on the host: one entry per sequence of the batch."""
    slots: tuple       # cache slot of every sequence
    news: tuple        # tokens each brings in this step
    pasts: tuple       # tokens each had cached before
    starts: tuple      # [B + 1] offsets of the sequences among the step's token rows

    @property
    def n_tokens(self) -> int:
        return self.starts[-1]

    @property
    def n_seqs(self) -> int:
        return len(self.slots)


class Part:
    """Base of every part.  ``params`` maps tensor name -> the view the loader
    fills; it exists after ``allocate``."""

    # True: the part may run inside a captured step (see the module's text); parts from outside the
    # library are taken to be unsafe until they say otherwise
    graph_safe = False

    def param_specs(self) -> list:
        return []

    def step_arrays(self, step: "StepHost") -> dict:
        """name -> int32 numpy array that this part wants on the device for this
        step.  Names are global: parts that return the same name must mean the
        same list (the first one is kept)."""
        return {}

    def step_arrays_key(self):
        """Parts with equal keys would return the same lists; only one of them
        is asked.  None: this part has no lists."""
        return None

    def allocate(self, stored: dict, rt: "Runtime") -> dict:
        """``stored``: tensor name -> dtype in the checkpoint (only names that
        are present).  Returns tensor name -> destination view."""
        return {}

    def finalize(self) -> None:
        """Called once every view has been filled; device-side tables are built
        here, never in the constructor.  Must be harmless when called twice."""

    def children(self) -> list:
        return []


def plain_delta(norm, delta):
    """What a norm is given as ``delta``.  A producer may hand on a deferred
    output (an object with ``materialize()`` that also knows how to fold its
    last step into an add + norm); only a norm that says ``takes_deferred =
    True`` sees it, every other norm gets the plain tensor."""
    if hasattr(delta, "materialize") and not getattr(norm, "takes_deferred", False):
        return delta.materialize()
    return delta


def walk(part: Part):
    yield part
    for c in part.children():
        yield from walk(c)


# ---------------------------------------------------------------------------
# registries: spec.kind -> builder(spec, rt) -> part
# ---------------------------------------------------------------------------
_REGISTRIES: dict = {"mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}}


def register(family: str, kind: str, builder: Callable) -> None:
    if family not in _REGISTRIES:
        raise InvalidConfig(f"no part family {family!r}; families: {sorted(_REGISTRIES)}")
    _REGISTRIES[family][kind] = builder


def build(family: str, spec, rt: "Runtime"):
    if spec is None:
        return None
    kind = getattr(spec, "kind", None)
    builder = _REGISTRIES[family].get(kind)
    if builder is None:
        raise InvalidConfig(f"no {family} is registered under {kind!r}; registered: {sorted(_REGISTRIES[family])}")
    return builder(spec, rt)


# ---------------------------------------------------------------------------
# runtime
# ---------------------------------------------------------------------------
class Workspace:
    """Named scratch buffers that live as long as the runtime.  A buffer only
    grows; while ``frozen`` (a CUDA graph holds the addresses) growth is an error."""

    def __init__(self, device):
        self.device = device
        self._bufs: dict = {}
        self._views: dict = {}       # (name, dtype, shape) -> the view handed out last time (a step asks for the same ones)
        self.frozen = False
        self.generation = 0          # bumped whenever a buffer moves; captured graphs check it

    def get(self, name: str, shape: tuple, dtype) -> torch.Tensor:
        seen = self._views.get((name, dtype, shape))
        if seen is not None:
            return seen
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise Backend(f"workspace buffer {name} would have to grow while a captured graph holds it")
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if (k[0], k[1]) != key}    # views of the old buffer
        view = buf[:count].view(*shape)
        if len(self._views) < 4096:
            self._views[(name, dtype, shape)] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class Runtime:
    """Device, activation dtype, scratch and the device status word."""

    def __init__(self, device, dtype: torch.dtype, ffn_chunk_tokens: int = 16384):
        """``device`` None gives a runtime that can only enumerate parts and
        their parameters (used to write model folders without a GPU)."""
        if dtype not in (torch.float32, torch.bfloat16):
            raise InvalidConfig(f"dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.shared_parts: dict = {}
        self.device = None
        self.side_stream = None
        if device is not None:
            self.device = torch.device(device)
            if self.device.type != "cuda":
                raise Backend("esp_b200 runs on a CUDA device only; there is no CPU path")
            self.ws = Workspace(self.device)
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.side_stream = torch.cuda.Stream(device=self.device)     # for work that may run beside the main stream
            self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.ffn_chunk_tokens = ffn_chunk_tokens
        self.record_routing = False       # debugging aid: MoE parts put their choices into ctx.aux
        # named 64-bit counters that kernels add to on the device (read with ``read_counters``: that waits)
        self._counter_names: list = []
        self.counters = None
        if self.device is not None:
            self.counters = torch.zeros(self.MAX_COUNTERS, dtype=torch.int64, device=self.device)

    MAX_COUNTERS = 1024

    def new_counter(self, name: str):
        """A one-element int64 view that a part's kernels may add to; None on a
        runtime without a device."""
        if self.counters is None:
            return None
        if len(self._counter_names) >= self.MAX_COUNTERS:
            raise Backend(f"more than {self.MAX_COUNTERS} device counters were asked for")
        self._counter_names.append(name)
        i = len(self._counter_names) - 1
        return self.counters[i:i + 1]

    def read_counters(self) -> dict:
        """name -> value; names given more than once are summed."""
        if self.counters is None:
            return {}
        host = self.counters[:len(self._counter_names)].tolist()
        out: dict = {}
        for name, v in zip(self._counter_names, host):
            out[name] = out.get(name, 0) + int(v)
        return out

    @property
    def full_precision(self) -> bool:
        return self.dtype == torch.float32

    def matrix_dtype(self, stored_dtypes) -> torch.dtype:
        """Dtype a (packed) weight matrix is kept in: in the 32-bit engine
        everything is widened to float32 (exact); otherwise bfloat16 stays
        bfloat16 and anything stored wider stays 32-bit."""
        if self.full_precision:
            return torch.float32
        return torch.bfloat16 if all(d == torch.bfloat16 for d in stored_dtypes) else torch.float32


@dataclass
class StepContext:
    """Everything about one step that parts may need.  All index tensors are
    int32 on the device."""
    n_tokens: int
    n_seqs: int
    max_new: int                     # longest run of new tokens of one sequence
    max_len: int                     # longest sequence after the step
    tok_ids: torch.Tensor            # [N]
    tok_seq: torch.Tensor            # [N] index of the token's sequence within the step
    tok_pos: torch.Tensor            # [N] absolute position of the token in its sequence
    seq_slot: torch.Tensor           # [B] cache slot of each sequence
    seq_start: torch.Tensor          # [B+1] offsets of the sequences in the token rows
    seq_past: torch.Tensor           # [B] cached length before the step
    want_rows: torch.Tensor          # [R] token rows whose logits are wanted
    block_tables: list               # per layer group: [B, stride] page ids
    host: dict                       # the same lists on the host (slots, starts, pasts, news); not for graph-safe parts
    aux: dict
    arrays: dict = field(default_factory=dict)    # name -> device tensor of every list the parts asked for (step_arrays)
