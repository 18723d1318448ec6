"""The generation loop above the step function.

Rules taken from the reference's loop
(crates/esp/src/infer/decoder/generate.rs:134-170,
crates/esp/src/infer/decoder/provider.rs:474-517): an empty prompt and
``max_tokens == 0`` are errors; a prompt as long as the context window is too
long; ``max_new = min(max_tokens, window - prompt)``; a stop token ends the
sequence, is not emitted and still costs its draw; after a token is kept the
callback may stop the sequence; the forward pass after the last token is
skipped.

What the reference does not have: batches.  Requests are packed into batches
that start together; prompts of unequal lengths run in one step, then every
live sequence advances by one token per step; a sequence that ends leaves the
batch and gives its slot back at once; batches follow one another until every
request is served.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from ..cache.book import PAGE
from ..errors import Backend, CacheFull, InvalidRequest, NonFiniteScores, PromptTooLong
from ..sampling.sampler import skip_draws
from ..sampling import SamplingParams


@dataclass
class SequenceRequest:
    """One request at the token seam."""
    prompt_ids: list
    max_tokens: int = 256
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: tuple = ()


@dataclass
class SequenceResult:
    token_ids: list
    finish_reason: str            # "stop" (stop token), "length" (budget) or "cancelled" (callback)
    prompt_tokens: int
    seed: Optional[int] = None    # the seed the stream was started from (sampled requests)


@dataclass
class ScoreHealth:
    """What the loop saw of the logits' health, as the reference counts it
    (crates/esp/src/infer/decoder/provider.rs:34-60).  The device checks a step's
    rows together, so ``invalid_steps`` counts steps, not rows."""
    checked_rows: int = 0
    invalid_steps: int = 0
    prefix_recomputations: int = 0
    failed_recoveries: int = 0


def budget(prompt_len: int, max_tokens: int, window: int) -> int:
    """Tokens a request may generate; raises as the reference does."""
    if prompt_len == 0:
        raise InvalidRequest("the prompt is empty")
    if max_tokens <= 0:
        raise InvalidRequest("max_tokens must be positive")
    if prompt_len >= window:
        raise PromptTooLong(prompt_len, window)
    return min(max_tokens, window - prompt_len)


def reserved_tokens(prompt_len: int, max_new: int) -> int:
    """Cache tokens a sequence can come to hold, rounded up to whole pages.  The
    last generated token is never fed back, so it needs no room."""
    held = prompt_len + max_new - 1
    return (max(held, 1) + PAGE - 1) // PAGE * PAGE


def form_batches(lengths: list, max_batch: int, max_tokens: int) -> list:
    """Splits requests, in order, into batches of at most ``max_batch``
    sequences whose reserved tokens fit ``max_tokens``.  ``lengths``: one
    (prompt_len, max_new) per request.  Returns lists of request indices."""
    batches, cur, used = [], [], 0
    for i, (p, m) in enumerate(lengths):
        need = reserved_tokens(p, m)
        if need > max_tokens:
            raise InvalidRequest(f"request {i} needs room for {need} tokens, the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    """Drives a backend with four calls:

    ``open(sampling, seed) -> slot``, ``close(slot)``,
    ``prefill(slots, prompts) -> tokens`` (one chosen token per sequence) and
    ``decode(slots, tokens) -> tokens``.  The backend chooses tokens on the
    device with each slot's own sampling options; this class only decides what
    runs next and what is kept."""

    def __init__(self, backend, window: int, max_batch: int, max_tokens: int, default_stop_ids=(),
                 health: Optional[ScoreHealth] = None):
        self.backend = backend
        self.window = window
        self.max_batch = max_batch
        self.max_tokens = max_tokens
        self.default_stop_ids = tuple(default_stop_ids)
        self.health = health if health is not None else ScoreHealth()
        self._recovery_used = False

    # A corrupt row of scores must never become a token.  When the backend reports non-finite
    # scores (NonFiniteScores), the tokens of that step are thrown away and the committed prefix of
    # every live sequence (prompt + tokens kept so far) is run again from fresh slots, once per
    # ``run`` call; if scores are bad again, or a second time later in the call, the call fails with
    # Backend (crates/esp/src/infer/decoder/provider.rs:219-240, :763-803).  Each sequence's sampling
    # stream restarts where it stood before the failed step, so draws are unchanged.
    def _recover(self, live, slots, seeds, outs, requests, launch):
        """Closes the live sequences' slots, opens fresh ones and returns
        ``launch(slots, prefixes)``: the re-run of the committed prefixes."""
        self.health.invalid_steps += 1
        if self._recovery_used:
            self.health.failed_recoveries += 1
            raise Backend("non-finite model scores after numerical recovery was already used")
        self._recovery_used = True
        self.health.prefix_recomputations += 1
        if hasattr(self.backend, "settle"):
            self.backend.settle()
        for i in live:
            self.backend.close(slots.pop(i))
        for i in live:
            seed = seeds[i]
            if seed is not None:
                seed = skip_draws(seed, len(outs[i]))        # one draw per kept token went before
            slots[i] = self.backend.open(requests[i].sampling, seed)
        prefixes = [list(requests[i].prompt_ids) + list(outs[i]) for i in live]
        try:
            return launch([slots[i] for i in live], prefixes)
        except NonFiniteScores:
            self.health.invalid_steps += 1
            self.health.failed_recoveries += 1
            raise Backend("recomputed model scores are non-finite") from None

    def run(self, requests: list, on_token: Optional[Callable] = None) -> list:
        """``on_token(request_index, token) -> bool``: a true return value
        stops that sequence after the token is kept."""
        self._recovery_used = False
        budgets = []
        for r in requests:
            r.sampling.validate()
            budgets.append(budget(len(r.prompt_ids), r.max_tokens, self.window))
        results = [None] * len(requests)
        lengths = [(len(r.prompt_ids), b) for r, b in zip(requests, budgets)]
        for batch in form_batches(lengths, self.max_batch, self.max_tokens):
            self._run_batch(batch, requests, budgets, results, on_token)
        return results

    def _run_batch(self, batch, requests, budgets, results, on_token):
        if hasattr(self.backend, "decode_async"):
            return self._run_batch_ahead(batch, requests, budgets, results, on_token)
        slots, seeds, outs = {}, {}, {}
        live = []
        try:
            for i in batch:
                seed = None if requests[i].sampling.greedy else requests[i].sampling.resolved_seed()
                seeds[i] = seed
                slots[i] = self.backend.open(requests[i].sampling, seed)
                outs[i] = []
                live.append(i)
            try:
                tokens = self.backend.prefill([slots[i] for i in live], [list(requests[i].prompt_ids) for i in live])
            except NonFiniteScores:
                tokens = self._recover(live, slots, seeds, outs, requests, self.backend.prefill)
            self.health.checked_rows += len(live)
            while live:
                nxt, feed = [], []
                for i, tok in zip(live, tokens):
                    tok = int(tok)
                    stops = self.default_stop_ids + tuple(requests[i].stop_token_ids)
                    reason = None
                    if tok in stops:
                        reason = "stop"
                    else:
                        outs[i].append(tok)
                        if on_token is not None and on_token(i, tok):
                            reason = "cancelled"
                        elif len(outs[i]) == budgets[i]:
                            reason = "length"
                    if reason is None:
                        nxt.append(i)
                        feed.append(tok)
                    else:
                        results[i] = SequenceResult(outs[i], reason, len(requests[i].prompt_ids), seeds[i])
                        self.backend.close(slots.pop(i))
                live = nxt
                if live:
                    try:
                        tokens = self.backend.decode([slots[i] for i in live], feed)
                    except NonFiniteScores:
                        # the fed tokens were kept already: they are part of the prefix that runs again
                        tokens = self._recover(live, slots, seeds, outs, requests, self.backend.prefill)
                    self.health.checked_rows += len(live)
        finally:
            for s in slots.values():      # only reached with slots left over when something raised
                self.backend.close(s)

    def _settle(self, i, tok, requests, budgets, outs, on_token):
        """What a chosen token means for its sequence: the reason it ends, or None."""
        stops = self.default_stop_ids + tuple(requests[i].stop_token_ids)
        if tok in stops:
            return "stop"
        outs[i].append(tok)
        if on_token is not None and on_token(i, tok):
            return "cancelled"
        if len(outs[i]) == budgets[i]:
            return "length"
        return None

    def _run_batch_ahead(self, batch, requests, budgets, results, on_token):
        """The same decisions with the backend one step ahead: the next decode
        step is launched, with its tokens taken on the device, before the host
        reads the tokens of this one.  Whether a sequence ends by its budget is
        known beforehand; a stop token or the caller's wish to stop is not, so a
        sequence that ends that way has one more row computed, which is thrown
        away (rows of a batch do not depend on each other)."""
        slots, seeds, outs = {}, {}, {}
        try:
            for i in batch:
                seed = None if requests[i].sampling.greedy else requests[i].sampling.resolved_seed()
                seeds[i] = seed
                slots[i] = self.backend.open(requests[i].sampling, seed)
                outs[i] = []
            order = list(batch)                          # whose token stands where in the step being waited for
            handle = self.backend.prefill_async([slots[i] for i in order], [list(requests[i].prompt_ids) for i in order])
            while handle is not None:
                # those that go on unless their token, still on its way, ends them
                ahead = [i for i in order if i in slots and len(outs[i]) + 1 < budgets[i]]
                nxt = None
                if ahead:
                    try:
                        nxt = self.backend.decode_async([slots[i] for i in ahead], handle, [order.index(i) for i in ahead])
                    except CacheFull:
                        nxt = None                       # a page for a row that may not be needed: decide after the tokens
                try:
                    tokens = handle.result()
                except NonFiniteScores:
                    # the step launched ahead took its tokens from the bad step: it is dropped with it
                    order = [i for i in order if i in slots]
                    handle = self._recover(order, slots, seeds, outs, requests, self.backend.prefill_async)
                    try:
                        tokens = handle.result()
                    except NonFiniteScores:
                        self.health.invalid_steps += 1
                        self.health.failed_recoveries += 1
                        raise Backend("recomputed model scores are non-finite") from None
                    nxt = None
                self.health.checked_rows += len(order)
                for i, tok in zip(order, tokens):
                    if i not in slots:
                        continue                         # ended a step ago: this row was computed for nothing
                    reason = self._settle(i, int(tok), requests, budgets, outs, on_token)
                    if reason is not None:
                        results[i] = SequenceResult(outs[i], reason, len(requests[i].prompt_ids), seeds[i])
                        self.backend.close(slots.pop(i))
                if nxt is None:
                    ahead = [i for i in order if i in slots]
                    if ahead:
                        nxt = self.backend.decode_async([slots[i] for i in ahead], handle, [order.index(i) for i in ahead])
                handle, order = nxt, ahead
        finally:
            for s in slots.values():      # only reached with slots left over when something raised
                self.backend.close(s)
