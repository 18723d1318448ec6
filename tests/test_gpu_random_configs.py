"""Configurations drawn at random from the sizes the architecture allows (tests/tiny.py: random_config), each
with random weights: the engine against the plain implementation under three cuttings in both dtypes; the
32-bit cuttings bit for bit with captured steps; generation through the entry point against the plain loop."""
import numpy as np
import pytest

import plain_qwen2_moe as plain
from gpu_util import Recorder, check_against_plain, run_steps, steps_batches, steps_tail, steps_whole
from tiny import random_config, random_ids

pytestmark = pytest.mark.gpu


def _folder(tmp_path, seed):
    from esp_b200.config import config_from_dict
    from esp_b200.weights import InitSpec, write_model_folder
    rng = np.random.default_rng(seed)
    raw = random_config(rng)
    folder = tmp_path / f"drawn_{seed}"
    write_model_folder(config_from_dict(raw), seed, folder, "bfloat16", InitSpec(0.05, 0.03, 0.02))
    return raw, folder, rng


def _folder_with(tmp_path, seed, **overrides):
    from esp_b200.config import config_from_dict
    from esp_b200.weights import InitSpec, write_model_folder
    rng = np.random.default_rng(seed)
    raw = dict(random_config(rng), **overrides)
    folder = tmp_path / f"drawn_{seed}"
    write_model_folder(config_from_dict(raw), seed, folder, "bfloat16", InitSpec(0.05, 0.03, 0.02))
    return raw, folder, rng


@pytest.mark.parametrize("seed, head_dim", [(24, None), (25, None), (26, None), (27, None), (28, None), (29, None),
                                            (30, None), (31, None), (32, None), (33, None), (34, None), (35, None),
                                            (7000, 96), (7001, 112), (7002, 144), (7003, 192), (7004, 256)])
def test_drawn_configuration_against_plain(tmp_path, seed, head_dim):
    """``head_dim`` given: the drawn configuration with that head size (every multiple of 16 up to 256 runs: the
    split-key kernel takes 64, 128, 192 and 256, the tensor-memory prefill 64 and 128, the mma.sync prefill up to
    128, the plain kernel the rest)."""
    from esp_b200.engine import Engine
    raw, folder, rng = _folder_with(tmp_path, seed, **({"head_dim": head_dim} if head_dim else {}))
    lens = [int(x) for x in rng.integers(1, 260, size=3)] + [int(rng.integers(260, 700))]
    reqs = {f"r{i}": random_ids(rng, n, raw["vocab_size"]) for i, n in enumerate(lens)}
    c, w = plain.load_model(folder)
    sparse = any(plain.layer_is_moe(c, i) for i in range(c["num_hidden_layers"]))
    # a model without a sparse layer has no expert choices to compare: the check then takes none
    model = (c, w) if sparse else (dict(c, num_experts_per_tok=c["num_experts"]), w)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048)
        eng.rt.record_routing = True
        prompt_lens = {r: max(1, len(t) - int(rng.integers(0, 12))) for r, t in reqs.items()}
        for name, steps in (("whole", steps_whole(reqs)), ("last 20 one by one", steps_tail(reqs, 20)),
                            ("batches", steps_batches(reqs, [["r0", "r1", "r2"], ["r3", "r0"]], prompt_lens))):
            rec = Recorder(raw["vocab_size"])
            run_steps(eng, steps, rec)
            check_against_plain(model, dtype, reqs, rec, f"drawn configuration {seed}, {name}: {raw}")


@pytest.mark.parametrize("seed", range(6))
def test_drawn_configuration_cuttings_and_generation(tmp_path, seed):
    from esp_b200.engine import Engine
    from esp_b200.provider import DecoderProvider, GenerationRequest
    raw, folder, rng = _folder(tmp_path, 1000 + seed)
    lens = [int(x) for x in rng.integers(34, 200, size=4)]
    reqs = {f"r{i}": random_ids(rng, n, raw["vocab_size"]) for i, n in enumerate(lens)}
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024)
    eng.rt.record_routing = False                      # decode steps are captured and replayed
    outs = []
    for steps in (steps_whole(reqs), steps_tail(reqs, 32),
                  steps_batches(reqs, [["r0", "r1", "r2"], ["r3", "r0"]], {r: len(t) - 30 for r, t in reqs.items()})):
        rec = Recorder(raw["vocab_size"])
        run_steps(eng, steps, rec)
        outs.append(rec)
    for rid, toks in reqs.items():
        tail = list(range(len(toks) - 30, len(toks)))
        whole, one_by_one, batched = (o.logits_of(rid, tail) for o in outs)
        assert np.array_equal(whole, one_by_one) and np.array_equal(whole, batched), (seed, rid, raw)
    del eng
    c, w = plain.load_model(folder)
    prov = DecoderProvider.load(folder, dtype="float32", max_batch=3, max_tokens=1024)
    asks = [dict(prompt=random_ids(rng, int(rng.integers(1, 40)), raw["vocab_size"]), max_new=int(rng.integers(1, 12)),
                 temperature=float(rng.choice([0.0, 0.0, 0.9])), top_p=[None, 0.8][int(rng.integers(0, 2))],
                 seed=int(rng.integers(0, 2 ** 31)), stop=[int(rng.integers(0, raw["vocab_size"]))]) for _ in range(5)]
    got = prov.generate([GenerationRequest(prompt_ids=a["prompt"], max_tokens=a["max_new"], temperature=a["temperature"],
                                           top_p=a["top_p"] if a["temperature"] > 0 else None, seed=a["seed"],
                                           stop_token_ids=a["stop"]) for a in asks])
    for a, out in zip(asks, got):
        ref = plain.generate(c, w, a["prompt"], a["max_new"], eos=tuple(a["stop"]), temperature=a["temperature"],
                             top_p=a["top_p"] if a["temperature"] > 0 else None, seed=a["seed"])
        if a["temperature"] == 0.0:                   # a sampled token may differ where a mass lies within rounding of the draw
            assert out.token_ids == ref, (seed, raw)
