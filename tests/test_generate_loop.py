"""The generation loop's decisions, driven with a scripted backend (no GPU):
budgets, stop tokens, sequences that end earlier, slot hand-back, batches one
after another (rules: crates/esp/src/infer/decoder/generate.rs:134-170,
crates/esp/src/infer/decoder/provider.rs:474-517)."""
import pytest

from esp_b200.engine.generate import (GenerationLoop, SequenceRequest, budget, form_batches, reserved_tokens)
from esp_b200.errors import InvalidRequest, PromptTooLong
from esp_b200.sampling import SamplingParams, skip_draws, splitmix64_next


class ScriptedBackend:
    """Every sequence emits prompt[0], prompt[0]+1, ... ; records all calls."""

    def __init__(self, n_slots=4):
        self.free = list(range(n_slots))[::-1]
        self.held = {}
        self.calls = []
        self.max_live = 0

    def open(self, sampling, seed):
        s = self.free.pop()
        self.held[s] = None
        self.max_live = max(self.max_live, len(self.held))
        self.calls.append(("open", s, seed))
        return s

    def close(self, slot):
        assert slot in self.held, "closed twice"
        del self.held[slot]
        self.free.append(slot)
        self.calls.append(("close", slot))

    def prefill(self, slots, prompts):
        self.calls.append(("prefill", tuple(slots), tuple(len(p) for p in prompts)))
        for s, p in zip(slots, prompts):
            self.held[s] = p[0]
        return [self.held[s] for s in slots]

    def decode(self, slots, tokens):
        self.calls.append(("decode", tuple(slots), tuple(tokens)))
        for s, t in zip(slots, tokens):
            assert self.held[s] == t, "the loop fed back a token it was not given"
            self.held[s] = t + 1
        return [self.held[s] for s in slots]


def loop(backend, **kw):
    args = dict(window=64, max_batch=4, max_tokens=64 * 64, default_stop_ids=())
    args.update(kw)
    return GenerationLoop(backend, **args)


def test_budget_rules():
    assert budget(5, 256, 64) == 59 and budget(5, 10, 64) == 10
    with pytest.raises(InvalidRequest):
        budget(0, 10, 64)
    with pytest.raises(InvalidRequest):
        budget(5, 0, 64)
    with pytest.raises(PromptTooLong) as e:
        budget(64, 10, 64)            # a prompt of exactly the window is already too long
    assert (e.value.length, e.value.limit) == (64, 64)


def test_length_stop_and_skipped_last_forward():
    be = ScriptedBackend()
    (r,) = loop(be).run([SequenceRequest([10, 0, 0], max_tokens=3)])
    assert r.token_ids == [10, 11, 12] and r.finish_reason == "length" and r.prompt_tokens == 3
    # two decode steps only: the forward after the last token is skipped
    assert [c[0] for c in be.calls] == ["open", "prefill", "decode", "decode", "close"]


def test_stop_token_is_not_emitted_and_sequences_leave_early():
    be = ScriptedBackend()
    reqs = [SequenceRequest([10], max_tokens=8, stop_token_ids=(12,)),
            SequenceRequest([20, 1], max_tokens=5),
            SequenceRequest([12], max_tokens=5, stop_token_ids=(12,))]
    res = loop(be).run(reqs)
    assert res[0].token_ids == [10, 11] and res[0].finish_reason == "stop"
    assert res[1].token_ids == [20, 21, 22, 23, 24] and res[1].finish_reason == "length"
    assert res[2].token_ids == [] and res[2].finish_reason == "stop"
    decodes = [c for c in be.calls if c[0] == "decode"]
    assert [len(c[1]) for c in decodes] == [2, 2, 1, 1]           # the batch shrinks as sequences end
    closes = [i for i, c in enumerate(be.calls) if c[0] == "close"]
    first_decode = next(i for i, c in enumerate(be.calls) if c[0] == "decode")
    assert closes[0] < first_decode                                # a finished sequence gives its slot back at once
    assert not be.held


def test_default_stop_ids_and_callback_cancel():
    be = ScriptedBackend()
    seen = []

    def on_token(i, tok):
        seen.append((i, tok))
        return i == 1 and tok == 31
    res = loop(be, default_stop_ids=(13,)).run(
        [SequenceRequest([10], max_tokens=9), SequenceRequest([30], max_tokens=9)], on_token)
    assert res[0].token_ids == [10, 11, 12] and res[0].finish_reason == "stop"
    assert res[1].token_ids == [30, 31] and res[1].finish_reason == "cancelled"
    assert (1, 31) in seen and (0, 13) not in seen


def test_batches_follow_one_another_and_slots_are_used_again():
    be = ScriptedBackend(n_slots=2)
    reqs = [SequenceRequest([10 * i], max_tokens=2 + i % 3) for i in range(1, 8)]
    res = loop(be, max_batch=2).run(reqs)
    assert [r.token_ids[0] for r in res] == [10 * i for i in range(1, 8)]
    assert [len(r.token_ids) for r in res] == [2 + i % 3 for i in range(1, 8)]
    assert be.max_live == 2 and not be.held
    assert sum(c[0] == "prefill" for c in be.calls) == 4
    # no request joins a batch that has started: every prefill comes after the previous batch's last close
    opens = [c for c in be.calls if c[0] == "open"]
    assert len(opens) == 7


def test_batches_respect_the_cache_size():
    assert reserved_tokens(5, 1) == 64 and reserved_tokens(60, 6) == 128 and reserved_tokens(64, 1) == 64
    assert form_batches([(60, 6), (10, 10), (100, 100)], max_batch=8, max_tokens=256) == [[0, 1], [2]]
    with pytest.raises(InvalidRequest):
        form_batches([(300, 10)], 8, 256)


def test_requests_are_validated_before_anything_runs():
    be = ScriptedBackend()
    with pytest.raises(InvalidRequest):
        loop(be).run([SequenceRequest([1], 4), SequenceRequest([1], 4, SamplingParams(temperature=-1.0))])
    with pytest.raises(InvalidRequest):
        loop(be).run([SequenceRequest([1], 4, SamplingParams(temperature=float("nan")))])
    with pytest.raises(PromptTooLong):
        loop(be).run([SequenceRequest([1] * 64, 4)])
    assert be.calls == []


def test_seeds():
    be = ScriptedBackend()
    res = loop(be).run([SequenceRequest([1], 2, SamplingParams(0.8, None, 42)), SequenceRequest([1], 2),
                        SequenceRequest([1], 2, SamplingParams(0.8))])
    assert res[0].seed == 42 and res[1].seed is None and isinstance(res[2].seed, int)
    opens = [c for c in be.calls if c[0] == "open"]
    assert opens[0][2] == 42 and opens[1][2] is None
    state, first = splitmix64_next(0)
    assert first == 0xE220A8397B1DCDAF                 # public test vector of splitmix64 from seed 0
    three = splitmix64_next(splitmix64_next(state)[0])[0]
    assert skip_draws(0, 1) == state and skip_draws(0, 3) == three


def test_slots_are_closed_when_the_backend_fails():
    class Failing(ScriptedBackend):
        def decode(self, slots, tokens):
            raise RuntimeError("device lost")
    be = Failing()
    with pytest.raises(RuntimeError):
        loop(be).run([SequenceRequest([1], 4), SequenceRequest([2], 4)])
    assert not be.held


class AheadBackend(ScriptedBackend):
    """The same sequences through the calls that do not wait: a step's tokens are read only when the loop
    asks for them, and a decode step takes its tokens from the handle of the step before."""

    class Handle:
        def __init__(self, tokens):
            self.tokens = tokens
            self.read = False

        def result(self):
            self.read = True
            return list(self.tokens)

    def prefill_async(self, slots, prompts):
        return self.Handle(self.prefill(slots, prompts))

    def decode_async(self, slots, earlier, places):
        self.launched_before_read = getattr(self, "launched_before_read", 0) + (0 if earlier.read else 1)
        return self.Handle(self.decode(slots, [earlier.tokens[p] for p in places]))


@pytest.mark.parametrize("case", range(4))
def test_one_step_ahead_gives_the_same_results(case):
    """Stop tokens, budgets, a caller that stops a sequence, batches one after another: the loop that
    launches the next step before it reads this one's tokens ends every sequence as the waiting loop does."""
    cases = [
        [SequenceRequest([10, 0, 0], max_tokens=3)],
        [SequenceRequest([10], max_tokens=8, stop_token_ids=(12,)), SequenceRequest([20, 1], max_tokens=5),
         SequenceRequest([12], max_tokens=5, stop_token_ids=(12,))],
        [SequenceRequest([5 * i + 1] * (1 + i % 3), max_tokens=1 + (7 * i) % 5, stop_token_ids=(5 * i + 3,) if i % 2 else ())
         for i in range(11)],
        [SequenceRequest([30], max_tokens=6), SequenceRequest([40], max_tokens=6), SequenceRequest([50], max_tokens=1)],
    ]
    reqs = cases[case]

    def cancel(i, tok):
        return case == 3 and i == 1 and tok == 42            # the caller stops the second sequence at its third token

    plain, ahead = ScriptedBackend(), AheadBackend()
    want = loop(plain).run(reqs, cancel)
    got = loop(ahead).run(reqs, cancel)
    assert [(r.token_ids, r.finish_reason, r.prompt_tokens) for r in got] == \
           [(r.token_ids, r.finish_reason, r.prompt_tokens) for r in want]
    assert not ahead.held and sorted(ahead.free) == list(range(4)), "a slot was lost"
    assert ahead.max_live <= 4
    if any(len(r.token_ids) > 2 for r in want):
        assert ahead.launched_before_read > 0, "no step was launched ahead of the tokens of the one before"
    # a sequence that ends by a stop token or by the caller has had at most one row too many
    extra = sum(len(c[1]) for c in ahead.calls if c[0] == "decode") - sum(len(c[1]) for c in plain.calls if c[0] == "decode")
    ended_early = sum(r.finish_reason in ("stop", "cancelled") for r in want)
    assert 0 <= extra <= ended_early


def test_one_step_ahead_waits_when_the_cache_cannot_take_the_step_launched_ahead():
    """A step launched ahead may ask for a page for a row that turns out not to be needed.  When the cache
    refuses it, the loop reads the tokens first and launches the step for those that really go on."""
    from esp_b200.errors import CacheFull

    class Tight(AheadBackend):
        refused = 0

        def decode_async(self, slots, earlier, places):
            if not earlier.read and len(slots) > 1:        # no room for every row that might go on
                self.refused += 1
                raise CacheFull("no page for a step launched ahead")
            return super().decode_async(slots, earlier, places)

    reqs = [SequenceRequest([10], max_tokens=6, stop_token_ids=(12,)), SequenceRequest([20], max_tokens=6)]
    want = loop(ScriptedBackend()).run(reqs)
    be = Tight()
    got = loop(be).run(reqs)
    assert [(r.token_ids, r.finish_reason) for r in got] == [(r.token_ids, r.finish_reason) for r in want]
    assert be.refused > 0 and not be.held


# ---------------------------------------------------------------------------
# non-finite scores: the committed prefix runs again once, then the call fails
# (crates/esp/src/infer/decoder/provider.rs:219-240, :763-803, tests :944-1020)
# ---------------------------------------------------------------------------
class Counting(ScriptedBackend):
    """Every sequence continues its last token: [.., t] -> t + 1, whether the prefix comes as a prompt or
    token by token.  ``bad_calls``: indices (over prefill and decode calls together) whose scores are
    reported as non-finite after the step has run."""

    def __init__(self, bad_calls=(), **kw):
        super().__init__(**kw)
        self.bad_calls = set(bad_calls)
        self.n_calls = 0
        self.settled = 0

    def _maybe_fail(self):
        from esp_b200.errors import NonFiniteScores
        self.n_calls += 1
        if self.n_calls - 1 in self.bad_calls:
            raise NonFiniteScores("the device reported: non-finite logits")

    def settle(self):
        self.settled += 1

    def prefill(self, slots, prompts):
        self.calls.append(("prefill", tuple(slots), tuple(len(p) for p in prompts)))
        for s, p in zip(slots, prompts):
            self.held[s] = p[-1] + 1
        self._maybe_fail()
        return [self.held[s] for s in slots]

    def decode(self, slots, tokens):
        self.calls.append(("decode", tuple(slots), tuple(tokens)))
        for s, t in zip(slots, tokens):
            assert self.held[s] == t
            self.held[s] = t + 1
        self._maybe_fail()
        return [self.held[s] for s in slots]


class CountingAhead(Counting):
    class Handle:
        def __init__(self, tokens, error):
            self.tokens, self.error, self.read = tokens, error, False

        def result(self):
            self.read = True
            if self.error is not None:
                raise self.error
            return list(self.tokens)

    def _handle(self, fn, *args):
        from esp_b200.errors import NonFiniteScores
        try:
            return self.Handle(fn(*args), None)
        except NonFiniteScores as e:                     # the step ran; its bad scores show when the tokens are read
            return self.Handle([self.held[s] for s in args[0]], e)

    def prefill_async(self, slots, prompts):
        return self._handle(self.prefill, slots, prompts)

    def decode_async(self, slots, earlier, places):
        return self._handle(self.decode, slots, [earlier.tokens[p] for p in places])


def _recovery_requests():
    return [SequenceRequest([10], max_tokens=6, sampling=SamplingParams(0.7, None, 1234)),
            SequenceRequest([20, 21], max_tokens=3),
            SequenceRequest([30], max_tokens=8, stop_token_ids=(35,))]


@pytest.mark.parametrize("backend_class", [Counting, CountingAhead])
@pytest.mark.parametrize("bad_call", [0, 1, 3])
def test_bad_scores_once_run_the_committed_prefix_again(backend_class, bad_call):
    from esp_b200.engine.generate import ScoreHealth
    want = loop(backend_class()).run(_recovery_requests())
    be = backend_class(bad_calls=[bad_call])
    health = ScoreHealth()
    got = loop(be, health=health).run(_recovery_requests())
    assert [(r.token_ids, r.finish_reason) for r in got] == [(r.token_ids, r.finish_reason) for r in want]
    assert (health.invalid_steps, health.prefix_recomputations, health.failed_recoveries) == (1, 1, 0)
    assert be.settled == 1 and not be.held and sorted(be.free) == list(range(4))
    # the sampled sequence's stream restarts where it stood: its seed moved on by one draw per kept token
    reopened = [c for c in be.calls if c[0] == "open" and c[2] is not None][1:]
    for c in reopened:
        assert c[2] in [skip_draws(1234, n) for n in range(0, 7)], "the reopened stream is not a continuation"
    # the prefix that ran again is prompt + kept tokens: one prefill more than a clean run, of longer prompts
    prefills = [c for c in be.calls if c[0] == "prefill"]
    assert len(prefills) == 2 and all(a >= b for a, b in zip(prefills[1][2], prefills[0][2][-len(prefills[1][2]):]))


# with the loop one step ahead, call 2 is the step launched before call 1's bad scores were read; it is dropped
# with them, and the re-run of the prefix is call 3
@pytest.mark.parametrize("backend_class, bad_calls, message", [
    (Counting, (1, 4), "already used"), (Counting, (1, 2), "recomputed"),
    (CountingAhead, (1, 4), "already used"), (CountingAhead, (1, 3), "recomputed")])
def test_bad_scores_again_fail_the_call_and_free_every_slot(backend_class, bad_calls, message):
    from esp_b200.engine.generate import ScoreHealth
    from esp_b200.errors import Backend
    be = backend_class(bad_calls=bad_calls)
    health = ScoreHealth()
    with pytest.raises(Backend, match=message):
        loop(be, health=health).run(_recovery_requests())
    assert health.prefix_recomputations == 1 and health.failed_recoveries == 1 and health.invalid_steps == 2
    assert not be.held and sorted(be.free) == list(range(4))


def test_cache_size_for_the_requests_at_hand():
    """The command line sizes the cache from its requests: prompt plus what each may generate (the last token is
    never fed back), in whole pages, the largest batch of at most max_batch requests."""
    from esp_b200.provider import cache_tokens_for
    assert cache_tokens_for([5], 16, window=4096, max_batch=8) == 64
    assert cache_tokens_for([60, 10], 10, window=4096, max_batch=8) == 128 + 64
    assert cache_tokens_for([100] * 5, 200, window=4096, max_batch=2) == 2 * 320       # batches of two: 299 -> 320 each
    assert cache_tokens_for([4000], 1000, window=4096, max_batch=1) == 4096            # budget cut at the window
