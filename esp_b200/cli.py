"""Command line: ``python -m esp_b200 <command>``.

The reference has no generation command; the options here carry the names and
meanings of its request (crates/esp/src/infer/provider.rs:91-117):
``--max-tokens``, ``--temperature`` (0 = greedy), ``--top-p``, ``--seed``,
``--stop``.  ``generate`` takes a model folder (``--model``) or a configuration
whose model gets random weights from a seed (``--random-config``, ``--weights-seed``).
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(a) -> int:
    from .config import config_from_json
    from .provider import DecoderProvider, GenerationRequest, cache_tokens_for, load_tokenizer
    reqs = []
    for ids in a.prompt_ids or []:
        reqs.append(GenerationRequest(prompt_ids=_ids(ids), max_tokens=a.max_tokens, temperature=a.temperature,
                                      top_p=a.top_p, seed=a.seed, stop=a.stop or [], stop_token_ids=a.stop_token_id or []))
    if (a.model is None) == (a.random_config is None):
        print("give either --model DIR or --random-config FILE (with --weights-seed)", file=sys.stderr)
        return 2
    if a.prompt:
        tok = load_tokenizer(a.model) if a.model is not None else None
        if tok is None:
            print("text prompts need tokenizer.json in the model folder (and the tokenizers package); "
                  "give --prompt-ids", file=sys.stderr)
            return 2
        for text in a.prompt:
            reqs.append(GenerationRequest(prompt_ids=tok.encode(text, add_special_tokens=True).ids,
                                          max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p,
                                          seed=a.seed, stop=a.stop or [], stop_token_ids=a.stop_token_id or []))
    if not reqs:
        print("give at least one --prompt-ids or --prompt", file=sys.stderr)
        return 2
    # the cache is sized for the requests at hand (prompt + what each may generate, in whole pages),
    # not for the most the model could ever hold
    config = config_from_json(a.model if a.model is not None else a.random_config)
    window = config.plan().max_positions
    if a.max_context is not None:
        window = min(window, a.max_context)
    cache_tokens = a.cache_tokens or cache_tokens_for([len(r.prompt_ids) for r in reqs], a.max_tokens, window, a.max_batch)
    if a.model is not None:
        prov = DecoderProvider.load(a.model, dtype=a.dtype, device=a.device, max_batch=a.max_batch,
                                    max_context=a.max_context, max_tokens=cache_tokens)
    else:
        # weights made on the device from the configuration and the seed: the same values that
        # ``random-model`` with this seed writes into a folder
        from .weights import InitSpec
        prov = DecoderProvider.from_random(config, a.weights_seed, init=InitSpec(a.weight_std, a.bias_std, a.norm_std),
                                           dtype=a.dtype, device=a.device, max_batch=a.max_batch,
                                           max_context=a.max_context, max_tokens=cache_tokens, stored_dtype=a.store_dtype)
    if a.profile:
        # one eager prefill of the first request and one eager decode step of it, timed kernel by kernel
        from .engine import StepEntry
        eng = prov.engine
        ids = list(reqs[0].prompt_ids)
        for timed in (False, True):          # once untimed: the first launches load the kernels
            slot = eng.open()
            try:
                _logits, prefill = eng.profile_step([StepEntry(slot, ids, [len(ids) - 1])])
                _logits, decode = eng.profile_step([StepEntry(slot, [ids[-1]], [0])])
            finally:
                eng.close(slot)
        print(f"prefill of {len(ids)} tokens, by kernel:\n{prefill.table()}\n\none decode step, by kernel:\n{decode.table()}",
              file=sys.stderr)
    for i, g in enumerate(prov.generate(reqs)):
        print(json.dumps({"request": i, "token_ids": g.token_ids, "text": g.text, "finish_reason": g.finish_reason,
                          "prompt_tokens": g.prompt_tokens, "seed": g.seed}))
    return 0


def cmd_random_model(a) -> int:
    from .config import config_from_json
    from .weights import InitSpec, write_model_folder
    cfg = config_from_json(a.config)
    write_model_folder(cfg, a.weights_seed, a.out, a.store_dtype, InitSpec(a.weight_std, a.bias_std, a.norm_std))
    print(a.out)
    return 0


def cmd_build(a) -> int:
    from .csrc.build import build_all
    for p in build_all():
        print(p)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="esp_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    g.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    g.add_argument("--random-config", default=None,
                   help="instead of --model: a config.json (or a folder with one) whose model gets random weights")
    g.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights of --random-config")
    g.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="with --random-config: the dtype a folder of these weights would hold (as random-model)")
    g.add_argument("--weight-std", type=float, default=0.02)
    g.add_argument("--bias-std", type=float, default=0.0)
    g.add_argument("--norm-std", type=float, default=0.0)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated; repeat for a batch")
    g.add_argument("--prompt", action="append", help="text prompt (needs tokenizer.json); repeat for a batch")
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--stop", action="append", help="stop string (text level)")
    g.add_argument("--stop-token-id", type=int, action="append")
    g.add_argument("--max-batch", type=int, default=64)
    g.add_argument("--max-context", type=int, default=None)
    g.add_argument("--profile", action="store_true",
                   help="before generating, time one prefill and one decode step kernel by kernel (to stderr)")
    g.add_argument("--cache-tokens", type=int, default=None,
                   help="cache size in tokens (default: what these requests need)")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random-model", help="write a model folder with random weights from a config.json and a seed")
    r.add_argument("--config", required=True)
    r.add_argument("--weights-seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--weight-std", type=float, default=0.02)
    r.add_argument("--bias-std", type=float, default=0.0)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.set_defaults(fn=cmd_random_model)
    b = sub.add_parser("build", help="compile every kernel library now")
    b.set_defaults(fn=cmd_build)
    a = ap.parse_args(argv)
    from .errors import InferError
    try:
        return a.fn(a)
    except InferError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
