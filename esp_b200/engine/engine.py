"""The engine: a model, its cache and the one step function.

``step`` takes a batch of sequences, each with the tokens it brings now (a
whole prompt, one decoded token, or any run in between), runs exactly those
tokens as one packed batch from what the cache holds, appends their keys and
values, and returns the logits at the places asked for.  There is no padding:
token rows are packed back to back and every kernel works on rows.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ..cache import Cache
from ..cache.storage import STATE_RNG, STATE_WORDS
from ..csrc import ops
from ..sampling import as_signed64
from ..config import config_from_json
from ..errors import Backend, InvalidRequest, NonFiniteScores
from ..parts import Runtime, StepContext
from ..parts.base import StepHost
from ..weights import FolderSource, InitSpec, RandomSource, load_into
from .model import DecoderModel

GRAPH_STRIDE_PAGES = 8       # page tables of captured decode steps grow in steps of 8 pages (512 positions)
DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    if name not in DTYPES:
        raise InvalidRequest(f"dtype must be one of {sorted(DTYPES)}, got {name!r}")
    return DTYPES[name]


class PendingTokens:
    """Tokens of a step on their way to the host.  ``device`` is the step's own
    copy on the device (a later step may take its tokens from it), ``result()``
    waits for the copy to the host and returns the list."""

    def __init__(self, device: torch.Tensor, host: torch.Tensor, landed):
        self.device = device
        self._host = host
        self._landed = landed

    def result(self) -> list:
        self._landed.synchronize()
        return self._host.tolist()


@dataclass
class StepEntry:
    slot: int
    tokens: list
    want: list = field(default_factory=list)     # places among ``tokens`` whose logits are wanted


class Engine:
    def __init__(self, config, source_factory, dtype="bfloat16", device="cuda:0", max_tokens: int = 8192,
                 max_slots: Optional[int] = None, shrink_to_fit: bool = False):
        """``source_factory(specs) -> source``: gives the loader its tensors.
        ``max_tokens`` sizes the cache; it is refused if weights and cache do not
        fit the device's free memory, or, with ``shrink_to_fit``, made as small
        as fits (``self.max_tokens`` tells what it became)."""
        self.config = config
        self.plan = config.plan()
        self.dtype = parse_dtype(dtype)
        if not torch.cuda.is_available():
            raise Backend("no CUDA device is visible; esp_b200 has no CPU path")
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.rt = Runtime(device, self.dtype)
        with torch.cuda.device(self.rt.device):
            self.model = DecoderModel(self.plan, self.rt)
            specs = [s for part in self.model.all_parts() for s in part.param_specs()]
            source = source_factory(specs)
            self.memory_plan = self._check_memory(specs, source, max_tokens, shrink_to_fit)
            max_tokens = self.memory_plan["cache_tokens"]
            self.max_tokens = max_tokens
            load_into(self.model, source, self.rt)
            n_pages = (max_tokens + 63) // 64
            if max_slots is None:
                max_slots = max(1, min(n_pages, 4096))
            self.max_slots = max_slots
            self.cache = Cache(self.model.cache_requests(), max_tokens, max_slots, self.plan.max_positions,
                               self.dtype, self.rt.device)
        parts = self.model.all_parts()
        # a decode step is replayed from a captured graph only if every part says that it may be
        self._parts_graph_safe = all(getattr(p, "graph_safe", False) for p in parts)
        self._array_makers, seen = [], set()
        for p in parts:
            key = p.step_arrays_key()
            if key is not None and key not in seen:
                seen.add(key)
                self._array_makers.append(p)
        self._host_counters = {"steps": 0, "tokens": 0, "kv_bytes_read": 0}
        # testing aid: the index of a wanted logits row that is overwritten with NaN before the finite
        # check, to exercise what follows a failed check without a faulty model; ``poison_steps`` says for
        # how many more forward passes (None: until the row is set back to None)
        self.poison_logits_row: Optional[int] = None
        self.poison_steps: Optional[int] = None
        self._pinned = None
        self._pinned_event = None
        self._copy_stream = None
        self.staged_bytes = 0
        self._meta_dev = None
        self.steps_run = 0
        # decode steps (one token per sequence) are captured into CUDA graphs, one per
        # (batch size, page-table stride, what is wanted); see _run
        self.use_graphs = True
        self._graphs: dict = {}
        self._graph_seen: dict = {}
        self.graph_replays = 0

    def _check_memory(self, specs, source, max_tokens: int, shrink: bool) -> dict:
        """Bytes of weights and cache that this engine is about to allocate against
        the device's free memory; refuses with the numbers instead of dying inside
        an allocation.  ``ESP_B200_MEMORY_HEADROOM`` (bytes, default 2 GiB) is kept
        for scratch buffers and the CUDA context."""
        el = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2}
        have = set(source.names())
        weights = 0
        for sp in specs:
            if sp.name not in have:
                continue
            count = int(np.prod(sp.shape)) if sp.shape else 1
            kept = self.rt.matrix_dtype([source.dtype(sp.name)]) if sp.role == "matrix" else torch.float32
            weights += count * el.get(kept, 4)
        tokens = (max_tokens + 63) // 64 * 64
        per_token = 0
        for layout, _state, cache_of in self.model.cache_requests():
            if layout is not None and cache_of is None:
                per_token += 2 * layout.num_kv_heads * layout.head_dim * el[self.dtype]
        cache = per_token * tokens
        free, total = torch.cuda.mem_get_info(self.rt.device)
        headroom = int(os.environ.get("ESP_B200_MEMORY_HEADROOM", 2 << 30))
        if shrink and weights + cache + headroom > free and per_token > 0:
            tokens = max(0, (free - weights - headroom) // per_token) // 64 * 64
            cache = per_token * tokens
        plan = {"weights_bytes": weights, "cache_bytes": cache, "cache_tokens": tokens, "free_bytes": free,
                "total_bytes": total}
        if weights + cache + headroom > free or tokens <= 0:
            gb = lambda v: f"{v / 1e9:.1f} GB"
            raise Backend(f"the model does not fit the device: weights {gb(weights)} + a cache of {tokens} tokens "
                          f"{gb(cache)} + {gb(headroom)} of headroom exceed the {gb(free)} that are free "
                          f"(of {gb(total)}); ask for a smaller cache (max_tokens) or fewer sequences")
        return plan

    # -- construction ---------------------------------------------------------
    @classmethod
    def from_folder(cls, folder, **kw) -> "Engine":
        folder = Path(folder)
        config = config_from_json(folder)
        return cls(config, lambda specs: FolderSource(folder), **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, init: InitSpec = InitSpec(), stored_dtype=None, **kw) -> "Engine":
        dt = parse_dtype(kw.get("dtype", "bfloat16")) if stored_dtype is None else parse_dtype(stored_dtype)
        return cls(config, lambda specs: RandomSource(specs, seed, init, dt), **kw)

    # -- slots -----------------------------------------------------------------
    def open(self) -> int:
        with torch.cuda.device(self.rt.device):
            return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.book.length(slot)

    # -- the step ----------------------------------------------------------------
    def _stage(self, arrays: list):
        """Packs int32 arrays into one pinned buffer, copies it to the device in
        one transfer and returns device views in the same order."""
        offsets, total = [], 0
        for a in arrays:
            offsets.append(total)
            total += (a.size + 3) // 4 * 4          # keep every section 16-byte aligned
        total = max(total, 4)
        if self._pinned is None or self._pinned.numel() < total:
            cap = max(total, 1 << 16)
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
            self._pinned_event = None
        if self._pinned_event is not None:
            self._pinned_event.synchronize()         # the last copy out of the pinned buffer is done
        host = self._pinned.numpy()
        for a, off in zip(arrays, offsets):
            host[off:off + a.size] = a.reshape(-1)
        self._meta_dev[:total].copy_(self._pinned[:total], non_blocking=True)
        self.staged_bytes = 4 * total                # what the last step copied to the device
        self._pinned_event = torch.cuda.Event()
        self._pinned_event.record()
        return [self._meta_dev[off:off + a.size].view(a.shape) for a, off in zip(arrays, offsets)]

    def plan_step(self, entries: list):
        """Validates a step against the cache without changing anything and
        returns the host-side arrays."""
        if not entries:
            raise InvalidRequest("a step needs at least one entry")
        book = self.cache.book
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise InvalidRequest("a slot appears twice in one step")
        vocab = self.plan.vocab
        news, pasts, want_rows = [], [], []
        start = 0
        starts = [0]
        for e in entries:
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.ndim != 1 or toks.size == 0:
                raise InvalidRequest(f"slot {e.slot}: a step entry needs at least one token")
            if toks.min() < 0 or toks.max() >= vocab:
                raise InvalidRequest(f"slot {e.slot}: token ids must lie in [0, {vocab})")
            for w in e.want:
                if not 0 <= int(w) < toks.size:
                    raise InvalidRequest(f"slot {e.slot}: wanted place {w} is outside its {toks.size} tokens")
                want_rows.append(start + int(w))
            news.append(int(toks.size))
            pasts.append(book.length(e.slot))
            start += int(toks.size)
            starts.append(start)
        growth = dict(zip(slots, news))
        book.check_step(growth)
        return slots, news, pasts, starts, want_rows, growth

    def step(self, entries: list, aux: Optional[dict] = None) -> torch.Tensor:
        """Runs the entries' tokens as one batch; returns float32 logits
        [number of wanted places, vocab] in the order of the entries and of
        their ``want`` lists.  On a validation error nothing is changed."""
        logits, _ = self._run(entries, aux, [])
        # a replayed graph writes its logits into the same buffer every time: hand out a copy
        return logits.clone() if self._graphs else logits

    def step_and_pick(self, entries: list, temperatures: list, top_ps: list, aux: Optional[dict] = None, feed=None):
        """One step that ends with the choice of the next token of every entry
        (each entry must want exactly one place).  ``temperatures[i] == 0``
        chooses the arg-max, otherwise a draw from the slot's own stream;
        ``top_ps[i]`` None means no nucleus cut.  Returns (tokens, logits):
        tokens is an int32 device tensor [B + 1] whose last element is the
        device status word.

        ``feed`` = (picks, src): ``picks`` is an int32 device tensor of tokens
        chosen by an earlier step and ``src[i] >= 0`` says that entry i (of one
        token) takes ``picks[src[i]]`` instead of the token it names, so that a
        step can follow a step before the host has read the tokens."""
        if any(len(e.want) != 1 for e in entries):
            raise InvalidRequest("step_and_pick needs exactly one wanted place per entry")
        temps = np.asarray(temperatures, dtype=np.float32)
        tops = np.asarray([-1.0 if t is None else t for t in top_ps], dtype=np.float32)
        rows = np.asarray([e.slot * STATE_WORDS + STATE_RNG for e in entries], dtype=np.int32)
        extra = [temps.view(np.int32), tops.view(np.int32), rows]
        if feed is not None:
            picks, src = feed
            if len(src) != len(entries) or any(i >= 0 and len(e.tokens) != 1 for e, i in zip(entries, src)):
                raise InvalidRequest("a fed entry brings exactly one token, and every entry needs a source index")
            if any(i >= picks.shape[0] for i in src):
                raise InvalidRequest("a source index lies beyond the earlier step's tokens")
            extra.append(np.asarray(src, dtype=np.int32))
        logits, out = self._run(entries, aux, extra, pick=True, feed=None if feed is None else feed[0])
        return out, logits

    def fetch_async(self, tokens: torch.Tensor) -> "PendingTokens":
        """Starts the copy of a step's tokens to the host on a stream of its own
        and returns at once; ``result()`` waits for that copy only, not for
        steps launched since."""
        with torch.cuda.device(self.rt.device):
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream()
                self._fetch_ring = [torch.empty(self.cache.book.slots.n + 1, dtype=torch.int32, pin_memory=True)
                                    for _ in range(4)]
                self._fetch_turn = 0
            kept = tokens.clone()                     # a replayed graph writes its tokens into the same buffer every time
            done = torch.cuda.Event()
            done.record()
            host = self._fetch_ring[self._fetch_turn % len(self._fetch_ring)][:kept.shape[0]]
            self._fetch_turn += 1
            self._copy_stream.wait_event(done)
            with torch.cuda.stream(self._copy_stream):
                host.copy_(kept, non_blocking=True)
                landed = torch.cuda.Event()
                landed.record()
            return PendingTokens(kept, host, landed)

    def seed_slot(self, slot: int, seed: int) -> None:
        """Starts the slot's sampling stream from ``seed``."""
        self.cache.engine_state[slot, STATE_RNG] = as_signed64(seed)

    def _run(self, entries: list, aux, extra_arrays: list, pick: bool = False, feed=None):
        with torch.cuda.device(self.rt.device):
            slots, news, pasts, starts, want_rows, growth = self.plan_step(entries)
            book = self.cache.book
            receipts = book.reserve(growth)
            try:
                result = self._run_reserved(entries, aux, extra_arrays, pick, feed, slots, news, pasts, starts, want_rows,
                                            growth)
            except BaseException:
                book.cancel(receipts)              # the step did not run: its pages go back, lengths stay
                raise
            book.commit(growth)
            self.steps_run += 1
            return result

    def _run_reserved(self, entries, aux, extra_arrays, pick, feed, slots, news, pasts, starts, want_rows, growth):
        book = self.cache.book
        b, n = len(entries), starts[-1]
        decode = n == b
        tok_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        tok_seq = np.repeat(np.arange(b, dtype=np.int32), news)
        tok_pos = np.concatenate([np.arange(p, p + t, dtype=np.int32) for p, t in zip(pasts, news)])
        stride = self.cache.max_table_stride(slots, growth)
        graphable = (decode and self.use_graphs and self._parts_graph_safe and not self.rt.record_routing
                     and aux is None and self.poison_logits_row is None)
        if graphable:
            stride = (stride + GRAPH_STRIDE_PAGES - 1) // GRAPH_STRIDE_PAGES * GRAPH_STRIDE_PAGES
        tables = [np.asarray(g.table_rows(slots, stride), dtype=np.int32).reshape(b, stride)
                  for g in book.groups]
        # the lists that the model's parts want on the device for this step (the engine knows none of them)
        host = StepHost(tuple(slots), tuple(news), tuple(pasts), tuple(starts))
        named = {}
        for part in self._array_makers:
            for name, arr in part.step_arrays(host).items():
                named.setdefault(name, np.ascontiguousarray(arr, dtype=np.int32))
        names = sorted(named)
        fixed = [tok_ids, tok_seq, tok_pos, np.asarray(slots, dtype=np.int32), np.asarray(starts, dtype=np.int32),
                 np.asarray(pasts, dtype=np.int32), np.asarray(want_rows, dtype=np.int32)]
        dev = self._stage([*fixed, *tables, *[named[k] for k in names], *extra_arrays])
        nf, nt = len(fixed), len(fixed) + len(tables)
        if feed is not None:                      # token ids from the earlier step's choices, on the device
            ops.feed_tokens(dev[0], feed, dev[-1])
        ctx = StepContext(
            n_tokens=n, n_seqs=b, max_new=max(news), max_len=max(p + t for p, t in zip(pasts, news)),
            tok_ids=dev[0], tok_seq=dev[1], tok_pos=dev[2], seq_slot=dev[3], seq_start=dev[4], seq_past=dev[5],
            want_rows=dev[6], block_tables=list(dev[nf:nt]),
            host={"slots": slots, "news": news, "pasts": pasts, "starts": starts, "want_rows": want_rows},
            aux=aux if aux is not None else {}, arrays=dict(zip(names, dev[nt:nt + len(names)])))
        extra = dev[nt + len(names):]
        self._count_step(news, pasts)
        if graphable:
            key = (b, stride, pick, tuple(want_rows), tuple((k, named[k].size) for k in names))
            return self._run_decode_graph(ctx, extra, pick, key)
        return self._forward(ctx, extra, pick)

    def _count_step(self, news, pasts) -> None:
        """Host-side counters of the work a step asks for (what the kernels must read of the cache follows
        from lengths and windows alone)."""
        c = self._host_counters
        c["steps"] += 1
        c["tokens"] += sum(news)
        el = torch.empty((), dtype=self.dtype).element_size()
        for layout, members in zip(self.cache.layouts, self.cache.members):
            per_key = 2 * len(members) * layout.num_kv_heads * layout.head_dim * el
            seen = 0
            for p, t in zip(pasts, news):
                # the keys the sequence's last new token sees: every kernel streams a sequence's visible keys once
                last = p + t
                seen += last if layout.window is None else min(last, layout.window + t - 1)
            c["kv_bytes_read"] += seen * per_key

    def profile_step(self, entries: list):
        """Runs one step eagerly on one stream (no captured graph, the shared expert in line) and returns
        (logits, ``ops.LaunchProfile``): device time by kind of kernel for this step.  Library products
        (cuBLAS) appear in the share of the kernel that follows them."""
        graphs, side = self.use_graphs, self.rt.side_stream
        self.use_graphs, self.rt.side_stream = False, None
        try:
            with torch.cuda.device(self.rt.device), ops.LaunchProfile() as prof:
                logits = self.step(entries)
            return logits, prof
        finally:
            self.use_graphs, self.rt.side_stream = graphs, side

    def counters(self) -> dict:
        """Work done since the engine was made: ``steps``, ``tokens``, ``kv_bytes_read`` (bytes of keys and
        values that the steps' attention had to read), and what the parts counted on the device
        (``expert_reads``: experts with at least one token, summed over sparse layers and steps).  Reading
        waits for the device."""
        out = dict(self._host_counters)
        out.update(self.rt.read_counters())
        return out

    def _forward(self, ctx, extra, pick: bool):
        logits = self.model.forward(ctx, self.cache)
        if self.poison_logits_row is not None and logits.shape[0] > self.poison_logits_row:
            logits[self.poison_logits_row].fill_(float("nan"))
            if self.poison_steps is not None:
                self.poison_steps -= 1
                if self.poison_steps <= 0:
                    self.poison_logits_row = self.poison_steps = None
        if not pick:
            return logits, None
        b = ctx.n_seqs
        out = self.rt.ws.get("picked_tokens", (b + 1,), torch.int32)
        ops.finite_check(logits, self.rt.status)
        ops.pick_tokens(logits, extra[0].view(torch.float32), extra[1].view(torch.float32),
                        self.cache.engine_state.view(-1), extra[2], out)
        out[b:].copy_(self.rt.status)
        return logits, out

    def _run_decode_graph(self, ctx, extra, pick: bool, key):
        """The first step of a shape runs eagerly (it sizes the scratch buffers and
        loads the kernels), the second is captured, later ones replay the graph.
        Everything that changes from step to step (token ids, positions, page
        tables, sampling options) lives in the staged buffer, whose addresses a
        shape fixes, so a replay needs one host-to-device copy and one launch."""
        ws = self.rt.ws
        entry = self._graphs.get(key)
        if entry is not None and (entry[3] != ws.generation or entry[4] is not self._meta_dev):
            del self._graphs[key]
            entry = None
        if entry is not None:
            entry[0].replay()
            self.graph_replays += 1
            ops.add_launches(entry[5])
            return entry[1], entry[2]
        seen = self._graph_seen.get(key, 0)
        self._graph_seen[key] = seen + 1
        if seen == 0 or seen < 0:
            return self._forward(ctx, extra, pick)
        graph = torch.cuda.CUDAGraph()
        ws.frozen = True
        before = ops.launch_count()
        try:
            with torch.cuda.graph(graph):
                logits, out = self._forward(ctx, extra, pick)
        except (RuntimeError, Backend):
            # a shape that cannot be captured (scratch would have to grow, or the runtime refuses the
            # capture) keeps running eagerly; nothing ran during the failed capture
            ws.frozen = False
            self._graph_seen[key] = -(1 << 30)
            torch.cuda.synchronize()
            return self._forward(ctx, extra, pick)
        finally:
            ws.frozen = False
        kernels = ops.launch_count() - before      # this library's kernels in the graph (library products not counted)
        ops.add_launches(-kernels)                 # capturing runs nothing
        self._graphs[key] = (graph, logits, out, ws.generation, self._meta_dev, kernels)
        graph.replay()
        ops.add_launches(kernels)
        self.graph_replays += 1
        return logits, out

    def read_status(self) -> int:
        """The device status word (0: nothing went wrong); reading it waits
        for the device."""
        return int(self.rt.status.item())

    def raise_on_status(self) -> None:
        code = self.read_status()
        if code:
            names = {1: "non-finite router probabilities", 2: "non-finite logits", 4: "a bounded wait ran out",
                     8: "an index on the device was out of range",
                     16: "a kernel's shared memory was not aligned as its layout needs"}
            what = ", ".join(v for k, v in names.items() if code & k)
            self.rt.status.zero_()
            if code == 2:
                raise NonFiniteScores(f"the device reported: {what}")
            raise Backend(f"the device reported: {what}")

    def settle(self) -> None:
        """Waits for everything launched so far and clears the status word: what a
        caller does before it runs a failed step's work again."""
        torch.cuda.synchronize(self.rt.device)
        self.rt.status.zero_()
