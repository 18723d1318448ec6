"""Helpers shared by the GPU tests: engines over tiny model folders, the three
ways of cutting a request into steps, and comparison with the plain
implementation."""
import functools
import re

import numpy as np
import torch

import plain_qwen2_moe as plain
from esp_b200.engine import Engine, StepEntry

# Bounds on |engine - plain| per request, relative to the largest |logit| of
# the request.  float32: the reference project accepts 2e-5 absolute on logits
# of order 0.1 (architecture_tests.rs:237-247); different summation orders
# give up to 1.7e-6 on the models of this suite (sums of 2,048 to 5,632 terms),
# so 6e-6 is the bound.  bfloat16: activations are rounded to 8 bits of mantissa
# (eps = 2^-8) a handful of times per layer; the worst request of the suite is
# off by 1.5 eps, and 3 eps is the bound.
REL_TOL = {"float32": 6e-6, "bfloat16": 3 * 2.0 ** -8}
# A routing choice may differ from the plain one only between experts whose
# probabilities are this close (relative), i.e. within rounding of a tie.
ROUTE_MARGIN = {"float32": 1e-5, "bfloat16": 2e-2}

_engines = {}


def engine_for(folder, dtype, max_tokens=2048, record_routing=True):
    """``record_routing``: the engine notes its expert choices for the comparison with the plain
    implementation; that keeps decode steps out of captured graphs, so tests of the graphs turn it off."""
    key = (str(folder), dtype, max_tokens, record_routing)
    if key not in _engines:
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)
        eng.rt.record_routing = record_routing
        _engines[key] = eng
    return _engines[key]


@functools.lru_cache(maxsize=None)
def plain_model(folder):
    return plain.load_model(folder)


class Recorder:
    """Collects, per request, the logits rows by position and the engine's
    routing choices by (layer, position)."""

    def __init__(self, vocab):
        self.vocab = vocab
        self.logits = {}
        self.routing = {}

    def take(self, entries, ids_of, logits, aux):
        """entries: [(rid, first_position, n_tokens, want)], in step order."""
        lg = logits.detach().float().cpu().numpy()
        row = 0
        for rid, first, n, want in entries:
            for w in want:
                self.logits.setdefault(rid, {})[first + w] = lg[row]
                row += 1
        assert row == lg.shape[0]
        for prefix, row0, ids, _w, _p in aux.get("routing", []):
            layer = int(re.search(r"layers\.(\d+)\.", prefix).group(1))
            ids = ids.cpu().numpy()
            start = 0
            for rid, first, n, _want in entries:
                lo, hi = max(start, row0), min(start + n, row0 + ids.shape[0])
                for r in range(lo, hi):
                    self.routing.setdefault(rid, {}).setdefault(layer, {})[first + (r - start)] = ids[r - row0]
                start += n

    def logits_of(self, rid, positions):
        return np.stack([self.logits[rid][p] for p in positions])

    def forced(self, rid, length):
        out = {}
        for layer, by_pos in self.routing.get(rid, {}).items():
            out[layer] = np.stack([by_pos[p] for p in range(length)])
        return out


def run_steps(engine, steps, recorder):
    """steps: list of (entries, end) with entries [(rid, tokens, want)]."""
    slots, pos = {}, {}
    for entries, end in steps:
        es, meta = [], []
        for rid, tokens, want in entries:
            if rid not in slots:
                slots[rid] = engine.open()
                pos[rid] = 0
            es.append(StepEntry(slots[rid], tokens, want))
            meta.append((rid, pos[rid], len(tokens), want))
            pos[rid] += len(tokens)
        if es:
            # a step that is asked to record is never replayed from a graph: ask only where the engine records
            aux = {} if engine.rt.record_routing else None
            logits = engine.step(es, aux)
            recorder.take(meta, None, logits, aux or {})
        for rid in end:
            engine.close(slots.pop(rid))
    assert not slots, "the trace left requests open"
    assert engine.read_status() == 0


def steps_whole(requests):
    return [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in requests.items()]


def steps_tail(requests, tail=32):
    steps = []
    for rid, toks in requests.items():
        cut = max(1, len(toks) - tail)
        steps.append(([(rid, toks[:cut], list(range(cut)))], []))
        for i in range(cut, len(toks)):
            steps.append(([(rid, [toks[i]], [0])], [rid] if i == len(toks) - 1 else []))
        if cut == len(toks):
            steps[-1] = (steps[-1][0], [rid])
    return steps


def steps_batches(requests, batches, prompt_lens):
    """Each batch starts its requests together with prompts of unequal lengths,
    then every live request goes on by one token; a request whose tokens are
    used up ends (named in ``end``) while the others go on."""
    steps = []
    for batch in batches:
        at = {rid: prompt_lens[rid] for rid in batch}
        first = [(rid, requests[rid][:at[rid]], list(range(at[rid]))) for rid in batch]
        steps.append((first, [rid for rid in batch if at[rid] == len(requests[rid])]))
        live = [rid for rid in batch if at[rid] < len(requests[rid])]
        while live:
            entries = [(rid, [requests[rid][at[rid]]], [0]) for rid in live]
            for rid in live:
                at[rid] += 1
            done = [rid for rid in live if at[rid] == len(requests[rid])]
            steps.append((entries, done))
            live = [rid for rid in live if rid not in done]
    return steps


def check_against_plain(folder, dtype, requests, recorder, what, positions=None):
    """``folder``: a model folder, or a loaded plain model (config, weights).  ``positions``: request id ->
    the positions to compare (default: all of them)."""
    c, w = folder if isinstance(folder, tuple) else plain_model(str(folder))
    k = c["num_experts_per_tok"]
    for rid, toks in requests.items():
        forced = recorder.forced(rid, len(toks))
        record = {}
        ref = plain.forward_logits(c, w, toks, forced_routing=forced, routing_record=record)
        at = list(range(len(toks))) if positions is None else list(positions[rid])
        got = recorder.logits_of(rid, at)
        ref = ref[at]
        scale = max(1e-6, float(np.abs(ref).max()))
        err = float(np.abs(got - ref).max())
        first_bad = at[int(np.argmax(np.abs(got - ref).max(axis=1) > REL_TOL[dtype] * scale))]
        assert err <= REL_TOL[dtype] * scale, (
            f"{what}, request {rid} ({len(toks)} tokens, {dtype}): max |engine - plain| = {err:.3e} > "
            f"{REL_TOL[dtype] * scale:.3e}; first wrong position {first_bad}")
        # the engine's expert choices are the plain ones up to rounding of near ties (an engine that recorded
        # none ran with the plain implementation's own choices: only sound where every expert is chosen)
        if not forced:
            assert k == c["num_experts"], "without the engine's expert choices only top-k = all experts can be compared"
            continue
        for layer, (ids_plain, p) in record.items():
            mine = forced[layer]
            for t in range(len(toks)):
                kth = np.sort(p[t])[-k]
                extra = set(int(e) for e in mine[t]) - set(int(e) for e in ids_plain[t])
                for e in extra:
                    assert p[t, e] >= kth * (1 - ROUTE_MARGIN[dtype]), (
                        f"{what}, request {rid}, layer {layer}, position {t}: the engine chose expert {e} "
                        f"(p={p[t, e]:.6f}) although the k-th probability is {kth:.6f}")
                assert len(set(int(e) for e in mine[t])) == k
