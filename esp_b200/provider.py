"""The Python entry point, in the vocabulary of the reference's provider seam
(crates/esp/src/infer/provider.rs:91-117, :263-325;
crates/esp/src/infer/decoder/provider.rs:263-343, :435-464, :522-559):
``GenerationRequest`` in, ``DecoderGeneration`` out, a ``DecoderProvider`` that
is loaded from a model folder (or made with random weights) and generates.

Differences from the reference: requests may carry token ids instead of text
(text needs ``tokenizer.json`` in the model folder and the ``tokenizers``
package), a call may hold several requests, which run as batches, and stop
token ids can be added per request.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Optional, Union

import torch

from .engine import Engine, StepEntry
from .engine.generate import GenerationLoop, ScoreHealth, SequenceRequest
from .errors import Backend, InvalidRequest, Unsupported
from .sampling import SamplingParams


@dataclass
class GenerationRequest:
    """One generation call's inputs; names and defaults as in the reference."""
    prompt: str = ""
    max_tokens: int = 256
    temperature: float = 0.0
    top_p: Optional[float] = None
    seed: Optional[int] = None
    stop: list = field(default_factory=list)            # stop strings (text level)
    prompt_ids: Optional[list] = None                   # token ids; take precedence over ``prompt``
    stop_token_ids: list = field(default_factory=list)  # extra stop tokens for this request


@dataclass
class DecoderGeneration:
    token_ids: list
    text: Optional[str]
    finish_reason: str
    prompt_tokens: int
    seed: Optional[int] = None


@dataclass(frozen=True)
class ModelCapability:
    context_window: int
    vocab_size: int
    architecture: str


class _EngineBackend:
    """What the generation loop drives: slots with their sampling options."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.options = {}

    def open(self, sampling: SamplingParams, seed):
        slot = self.engine.open()
        self.options[slot] = sampling
        if seed is not None:
            self.engine.seed_slot(slot, seed)
        return slot

    def close(self, slot):
        self.options.pop(slot, None)
        self.engine.close(slot)

    def settle(self):
        self.engine.settle()

    def _pick(self, entries):
        temps = [self.options[e.slot].temperature for e in entries]
        tops = [self.options[e.slot].top_p for e in entries]
        out, _ = self.engine.step_and_pick(entries, temps, tops)
        host = out.cpu().tolist()
        if host[-1]:
            self.engine.raise_on_status()
        return host[:-1]

    def prefill(self, slots, prompts):
        return self._pick([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])

    def decode(self, slots, tokens):
        return self._pick([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])

    # The same two calls without waiting for the tokens: they return a handle whose ``result()`` gives the
    # tokens, and a decode step takes its tokens on the device from the handle of the step before, so that it
    # can be launched before the host has read them.
    def _pick_async(self, entries, feed=None):
        temps = [self.options[e.slot].temperature for e in entries]
        tops = [self.options[e.slot].top_p for e in entries]
        out, _ = self.engine.step_and_pick(entries, temps, tops, feed=feed)
        return _StepHandle(self.engine, self.engine.fetch_async(out), len(entries))

    def prefill_async(self, slots, prompts):
        return self._pick_async([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])

    def decode_async(self, slots, earlier, places):
        """``places[i]``: where slot i's token stands among the tokens of ``earlier``."""
        return self._pick_async([StepEntry(s, [0], [0]) for s in slots], feed=(earlier.pending.device, list(places)))


class _StepHandle:
    def __init__(self, engine, pending, n):
        self.engine, self.pending, self.n = engine, pending, n

    def result(self) -> list:
        host = self.pending.result()
        if host[self.n]:
            self.engine.raise_on_status()
        return host[:self.n]


class DecoderProvider:
    def __init__(self, engine: Engine, tokenizer=None, max_batch: int = 64):
        self.engine = engine
        self.tokenizer = tokenizer
        self.max_batch = max_batch
        self._backend = _EngineBackend(engine)
        self.score_health = ScoreHealth()      # counts over this provider's generate calls

    # -- construction -----------------------------------------------------------
    @classmethod
    def load(cls, model_dir, dtype="bfloat16", device="cuda:0", max_batch: int = 64, max_context: Optional[int] = None,
             max_tokens: Optional[int] = None) -> "DecoderProvider":
        """``max_context``: longest sequence to make room for (default: the
        model's).  ``max_tokens``: cache size in tokens; refused if it does not
        fit the device.  Default: room for max_batch sequences of max_context,
        at most 1M tokens and at most what the device's free memory holds
        beside the weights."""
        model_dir = Path(model_dir)
        from .config import config_from_json
        config = config_from_json(model_dir)
        fit = max_tokens is None
        max_tokens = cls._cache_tokens(config, max_batch, max_context, max_tokens)
        engine = Engine.from_folder(model_dir, dtype=dtype, device=device, max_tokens=max_tokens, shrink_to_fit=fit)
        return cls(engine, load_tokenizer(model_dir), max_batch)

    @classmethod
    def from_random(cls, config, seed: int = 0, init=None, dtype="bfloat16", device="cuda:0", max_batch: int = 64,
                    max_context: Optional[int] = None, max_tokens: Optional[int] = None,
                    stored_dtype=None) -> "DecoderProvider":
        """Random weights made on the device.  ``stored_dtype``: the dtype a model
        folder of these weights would store them in (default: ``dtype``); with the
        same configuration, seed, ``init`` and stored dtype the values are those
        that ``write_model_folder`` writes."""
        from .weights import InitSpec
        fit = max_tokens is None
        max_tokens = cls._cache_tokens(config, max_batch, max_context, max_tokens)
        engine = Engine.from_random(config, seed, init or InitSpec(), stored_dtype=stored_dtype, dtype=dtype, device=device,
                                    max_tokens=max_tokens, shrink_to_fit=fit)
        return cls(engine, None, max_batch)

    @staticmethod
    def _cache_tokens(config, max_batch, max_context, max_tokens):
        if max_tokens is not None:
            return max_tokens
        window = config.plan().max_positions
        ctx = min(max_context or window, window)
        return min(max_batch * ((ctx + 63) // 64 * 64), 1 << 20)

    # -- what it can do ------------------------------------------------------------
    @property
    def capability(self) -> ModelCapability:
        p = self.engine.plan
        return ModelCapability(p.max_positions, p.vocab, p.architecture)

    def _ids(self, request: GenerationRequest) -> list:
        if request.prompt_ids is not None:
            return [int(t) for t in request.prompt_ids]
        if self.tokenizer is None:
            raise Unsupported("prompt", "text prompts need tokenizer.json in the model folder; pass prompt_ids")
        return self.tokenizer.encode(request.prompt, add_special_tokens=True).ids

    def generate(self, requests: Union[GenerationRequest, list],
                 on_token: Optional[Callable] = None) -> Union[DecoderGeneration, list]:
        """Generates for one request or for a list of them (run as batches of
        sequences that start together).  ``on_token(index, token) -> bool``
        may stop a sequence by returning true."""
        single = isinstance(requests, GenerationRequest)
        reqs = [requests] if single else list(requests)
        seqs = []
        for r in reqs:
            if r.stop and self.tokenizer is None:
                raise Unsupported("stop", "stop strings need a tokenizer; use stop_token_ids")
            seqs.append(SequenceRequest(self._ids(r), r.max_tokens, SamplingParams(r.temperature, r.top_p, r.seed),
                                        tuple(r.stop_token_ids)))
        hooks = self._stop_string_hook(reqs, on_token)
        loop = GenerationLoop(self._backend, self.engine.plan.max_positions, self.max_batch,
                              self.engine.cache.book.n_pages * 64, self.engine.plan.stop_token_ids,
                              health=self.score_health)
        results = loop.run(seqs, hooks)
        outs = []
        for r, res in zip(reqs, results):
            text = None
            if self.tokenizer is not None:
                text = self.tokenizer.decode(res.token_ids)
                for s in r.stop:
                    if s and s in text:
                        text = text[:text.index(s)]
            outs.append(DecoderGeneration(res.token_ids, text, res.finish_reason, res.prompt_tokens, res.seed))
        return outs[0] if single else outs

    def generate_streaming(self, request: GenerationRequest, on_token: Callable) -> DecoderGeneration:
        """One request; ``on_token(token) -> bool`` sees every kept token."""
        return self.generate(request, lambda _i, tok: bool(on_token(tok)))

    def _stop_string_hook(self, reqs, on_token):
        if not any(r.stop for r in reqs):
            return on_token
        seen = {i: [] for i in range(len(reqs))}

        def hook(i, tok):
            seen[i].append(tok)
            stop = bool(on_token(i, tok)) if on_token is not None else False
            if reqs[i].stop:
                text = self.tokenizer.decode(seen[i])
                stop = stop or any(s and s in text for s in reqs[i].stop)
            return stop
        return hook

    def next_token_logits(self, prompt_ids: list) -> torch.Tensor:
        """Float32 logits [vocab] after one prefill of ``prompt_ids`` with a
        fresh slot (crates/esp/src/infer/decoder/provider.rs:435-464)."""
        if not prompt_ids:
            raise InvalidRequest("the prompt is empty")
        slot = self.engine.open()
        try:
            logits = self.engine.step([StepEntry(slot, list(prompt_ids), [len(prompt_ids) - 1])])
            self.engine.raise_on_status()
            return logits[0]
        finally:
            self.engine.close(slot)


def load_tokenizer(model_dir):
    """The folder's tokenizer, or None if it has no tokenizer.json or the
    ``tokenizers`` package is missing (requests then carry token ids)."""
    path = Path(model_dir) / "tokenizer.json"
    if not path.is_file():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(str(path))


def cache_tokens_for(prompt_lengths: list, max_tokens: int, window: int, max_batch: int) -> int:
    """Cache size, in tokens, that serves these requests in batches of at most
    ``max_batch``: the largest batch's prompts plus what each may generate,
    every sequence rounded up to whole pages."""
    from .engine.generate import reserved_tokens
    need = [reserved_tokens(n, max(1, min(max_tokens, window - n))) for n in prompt_lengths]
    batches = [sum(need[i:i + max_batch]) for i in range(0, len(need), max_batch)]
    return max(batches, default=64)


def load(model_dir, **kw) -> DecoderProvider:
    return DecoderProvider.load(model_dir, **kw)
