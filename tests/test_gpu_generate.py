"""Generation through the Python entry point against the plain implementation:
greedy and seeded sampling, unequal prompts in one batch, stop tokens,
sequences that end earlier, batches that follow one another."""
import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from esp_b200.provider import DecoderProvider, GenerationRequest
from tiny import CASES, PROMPTS_A, PROMPTS_B, make_folder, random_ids

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    return {case: make_folder(tmp, case) for case in CASES}


def prompts(case, lengths, seed=5):
    rng = np.random.default_rng(seed)
    return [random_ids(rng, n, CASES[case][0]["vocab_size"]) for n in lengths]


def test_greedy_batch_of_unequal_prompts_float32(folders):
    """Tiny A: prompts of 5/11/17 tokens, 8 greedy tokens each, token by token."""
    prov = DecoderProvider.load(folders["A"], dtype="float32", max_batch=4)
    ps = prompts("A", PROMPTS_A)
    outs = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=8) for p in ps])
    c, w = plain.load_model(folders["A"])
    for p, o in zip(ps, outs):
        assert o.token_ids == plain.generate(c, w, p, 8) and o.finish_reason == "length" and o.prompt_tokens == len(p)
    # the same requests one batch after another (two at a time): same tokens, slots used again
    prov.max_batch = 2
    again = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=8) for p in ps])
    assert [o.token_ids for o in again] == [o.token_ids for o in outs]
    assert prov.engine.cache.book.slots.available == prov.engine.max_slots


def test_seeded_sampling_batch_float32(folders):
    """Tiny B: prompts of 1/7/23/40 tokens, 12 tokens at temperature 0.8."""
    prov = DecoderProvider.load(folders["B"], dtype="float32", max_batch=4)
    ps = prompts("B", PROMPTS_B)
    reqs = [GenerationRequest(prompt_ids=p, max_tokens=12, temperature=0.8, seed=100 + i) for i, p in enumerate(ps)]
    outs = prov.generate(reqs)
    c, w = plain.load_model(folders["B"])
    for i, (p, o) in enumerate(zip(ps, outs)):
        assert o.token_ids == plain.generate(c, w, p, 12, temperature=0.8, seed=100 + i), i
        assert o.seed == 100 + i
    assert [o.token_ids for o in prov.generate(reqs)] == [o.token_ids for o in outs], "same seed, same tokens"
    nucleus = prov.generate(GenerationRequest(prompt_ids=ps[2], max_tokens=12, temperature=0.8, top_p=0.3, seed=9))
    assert nucleus.token_ids == plain.generate(c, w, ps[2], 12, temperature=0.8, top_p=0.3, seed=9)
    unseeded = prov.generate(GenerationRequest(prompt_ids=ps[1], max_tokens=4, temperature=0.8))
    assert isinstance(unseeded.seed, int) and len(unseeded.token_ids) == 4
    assert unseeded.token_ids == plain.generate(c, w, ps[1], 4, temperature=0.8, seed=unseeded.seed)


def test_stop_tokens_and_early_ends(folders):
    prov = DecoderProvider.load(folders["A"], dtype="float32", max_batch=4)
    ps = prompts("A", PROMPTS_A, seed=8)
    c, w = plain.load_model(folders["A"])
    free = [plain.generate(c, w, p, 10) for p in ps]
    stop = free[1][3]                       # what request 1 would say fourth
    outs = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=10, stop_token_ids=[stop] if i == 1 else [])
                          for i, p in enumerate(ps)])
    cut = free[1].index(stop)
    assert outs[1].token_ids == free[1][:cut] and outs[1].finish_reason == "stop"
    assert outs[0].token_ids == free[0] and outs[2].token_ids == free[2]      # the others are not disturbed
    short = prov.generate([GenerationRequest(prompt_ids=ps[0], max_tokens=2), GenerationRequest(prompt_ids=ps[2], max_tokens=9)])
    assert short[0].token_ids == free[0][:2] and short[1].token_ids == free[2][:9]
    seen = []
    streamed = prov.generate_streaming(GenerationRequest(prompt_ids=ps[0], max_tokens=10), lambda t: seen.append(t) or len(seen) == 3)
    assert streamed.token_ids == free[0][:3] == seen and streamed.finish_reason == "cancelled"


@pytest.mark.parametrize("case", ["A", "B"])
def test_greedy_bfloat16_follows_the_plain_logits(folders, case):
    """In bfloat16 a near tie between two logits may fall the other way, so each
    chosen token is checked against the plain logits for the engine's own
    prefix: it must be the best token up to the bfloat16 bound."""
    prov = DecoderProvider.load(folders[case], dtype="bfloat16", max_batch=4)
    ps = prompts(case, PROMPTS_A if case == "A" else PROMPTS_B)
    outs = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=8) for p in ps])
    c, w = plain.load_model(folders[case])
    exact = 0
    for p, o in zip(ps, outs):
        assert len(o.token_ids) == 8
        ids = list(p)
        for tok in o.token_ids:
            row = plain.forward_logits(c, w, ids)[-1]
            assert row[tok] >= row.max() - 2 * 4 * 2.0 ** -8 * np.abs(row).max(), "not the best token within rounding"
            exact += int(tok == int(row.argmax()))
            ids.append(tok)
    assert exact >= 0.9 * 8 * len(ps)


def test_next_token_logits_and_capability(folders):
    prov = DecoderProvider.load(folders["B"], dtype="float32")
    p = prompts("B", [9])[0]
    c, w = plain.load_model(folders["B"])
    ref = plain.forward_logits(c, w, p)[-1]
    assert np.abs(prov.next_token_logits(p).cpu().numpy() - ref).max() < 2e-5 * max(1.0, np.abs(ref).max())
    cap = prov.capability
    assert (cap.context_window, cap.vocab_size, cap.architecture) == (256, 384, "Qwen2MoeForCausalLM")


def test_command_line_generates(folders, capsys):
    import json
    from esp_b200.cli import main
    p = prompts("A", [6])[0]
    rc = main(["generate", "--model", str(folders["A"]), "--dtype", "float32", "--prompt-ids", ",".join(map(str, p)),
               "--max-tokens", "5"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    c, w = plain.load_model(folders["A"])
    assert out["token_ids"] == plain.generate(c, w, p, 5) and out["finish_reason"] == "length"


def test_command_line_with_random_weights_equals_the_folder_of_the_same_seed(folders, tmp_path, capsys):
    """``generate --random-config`` makes on the device the weights that ``random-model`` with the same seed and
    deviations writes into a folder: the same tokens either way, and the tokens of the plain implementation."""
    import json
    from esp_b200.cli import main
    config = str(folders["B"] / "config.json")
    out = tmp_path / "written"
    spec = ["--weights-seed", "31", "--weight-std", "0.05", "--bias-std", "0.02", "--norm-std", "0.01"]
    assert main(["random-model", "--config", config, "--out", str(out)] + spec) == 0
    capsys.readouterr()
    p = prompts("B", [7, 19])
    ask = ["--dtype", "float32", "--max-tokens", "6"] + [x for q in p for x in ("--prompt-ids", ",".join(map(str, q)))]
    assert main(["generate", "--model", str(out)] + ask) == 0
    from_folder = [json.loads(line)["token_ids"] for line in capsys.readouterr().out.strip().splitlines()]
    assert main(["generate", "--random-config", config] + spec + ask) == 0
    from_seed = [json.loads(line)["token_ids"] for line in capsys.readouterr().out.strip().splitlines()]
    c, w = plain.load_model(out)
    assert from_folder == from_seed == [plain.generate(c, w, q, 6) for q in p]
    assert main(["generate"] + ask) == 2 and main(["generate", "--model", str(out), "--random-config", config] + ask) == 2


def test_waiting_and_one_step_ahead_agree_bfloat16(folders):
    """Seeded sampling in bfloat16 with a stop token and unequal budgets: the loop that launches the next step
    before it reads this one's tokens gives the tokens of the loop that waits, and hands every slot back."""
    from esp_b200.engine.generate import GenerationLoop, SequenceRequest
    from esp_b200.sampling import SamplingParams

    prov = DecoderProvider.load(folders["B"], dtype="bfloat16", max_batch=4)
    backend = prov._backend

    class Waiting:                                   # the same backend without the calls that do not wait
        open, close, prefill, decode = backend.open, backend.close, backend.prefill, backend.decode

    ps = prompts("B", PROMPTS_B, seed=11)
    window = prov.capability.context_window

    def run(be, stop):
        reqs = [SequenceRequest(p, max_tokens=6 + 3 * i, stop_token_ids=stop if i == 0 else (),
                                sampling=SamplingParams(temperature=0.9, top_p=0.8, seed=100 + i))
                for i, p in enumerate(ps)]
        return GenerationLoop(be, window, 4, 1 << 14).run(reqs)

    free = run(Waiting, ())
    stop = (free[0].token_ids[2],)
    want, got = run(Waiting, stop), run(backend, stop)
    assert [(r.token_ids, r.finish_reason) for r in got] == [(r.token_ids, r.finish_reason) for r in want]
    assert want[0].finish_reason == "stop" and len(want[0].token_ids) <= 2
    assert prov.engine.cache.book.slots.available == prov.engine.max_slots


def _poison_after(engine, steps_before, row=1, steps=1):
    """Arms the engine's testing aid so that the logits row ``row`` of the step number ``steps_before``
    (counted from now) is overwritten with NaN, and the same for ``steps`` steps in a row (None: for good)."""
    seen = {"n": 0}
    run_reserved = engine._run_reserved

    def counted(*args, **kw):
        if seen["n"] == steps_before:
            engine.poison_logits_row, engine.poison_steps = row, steps
        seen["n"] += 1
        return run_reserved(*args, **kw)

    engine._run_reserved = counted
    return lambda: setattr(engine, "_run_reserved", run_reserved)


@pytest.mark.parametrize("at", [0, 3])
def test_non_finite_logits_once_are_recomputed_and_change_nothing(folders, at):
    """A logits row turns NaN in one step (the prompts' step, or the third decode step): no token is taken
    from that step, the committed prefixes run again in fresh slots, and the tokens are those of a clean
    run, with seeded sampling too (the streams restart where they stood)."""
    prov = DecoderProvider.load(folders["B"], dtype="float32", max_batch=4)
    ps = prompts("B", PROMPTS_B, seed=21)
    reqs = [GenerationRequest(prompt_ids=p, max_tokens=9, temperature=0.0 if i % 2 else 0.8, seed=7 + i)
            for i, p in enumerate(ps)]
    clean = prov.generate(reqs)
    restore = _poison_after(prov.engine, at)
    try:
        again = prov.generate(reqs)
    finally:
        restore()
    assert [o.token_ids for o in again] == [o.token_ids for o in clean]
    h = prov.score_health
    assert (h.invalid_steps, h.prefix_recomputations, h.failed_recoveries) == (1, 1, 0) and h.checked_rows > 0
    assert prov.engine.cache.book.slots.available == prov.engine.max_slots
    assert all(g.pool.available == g.pool.n for g in prov.engine.cache.book.groups)
    assert prov.engine.read_status() == 0


def test_non_finite_logits_that_stay_fail_the_call_closed(folders):
    """Scores that are still bad after the one recomputation end the call with a Backend error that names
    them; no token of the bad steps is handed out, every slot and page goes back."""
    from esp_b200.errors import Backend
    prov = DecoderProvider.load(folders["A"], dtype="bfloat16", max_batch=4)
    ps = prompts("A", PROMPTS_A, seed=22)
    seen = []
    restore = _poison_after(prov.engine, 2, row=0, steps=None)
    try:
        with pytest.raises(Backend, match="non-finite"):
            prov.generate([GenerationRequest(prompt_ids=p, max_tokens=8) for p in ps], lambda i, t: seen.append((i, t)) and False)
    finally:
        restore()
        prov.engine.poison_logits_row = prov.engine.poison_steps = None
    assert max(sum(1 for i, _t in seen if i == r) for r in range(3)) <= 2, "tokens were taken from a step with bad scores"
    assert prov.score_health.failed_recoveries == 1
    assert prov.engine.cache.book.slots.available == prov.engine.max_slots
    assert all(g.pool.available == g.pool.n for g in prov.engine.cache.book.groups)
    prov.engine.settle()
    ok = prov.generate(GenerationRequest(prompt_ids=ps[0], max_tokens=3))      # the provider is still usable
    assert len(ok.token_ids) == 3


def test_profile_of_a_step_names_the_kernels_and_changes_nothing(folders, capsys):
    """``--profile`` / ``Engine.profile_step``: device time by kind of kernel for one eager step; the step's logits
    are those of the ordinary step, and generation afterwards is as without it."""
    from esp_b200.cli import main
    from esp_b200.engine import Engine, StepEntry
    eng = Engine.from_folder(folders["A"], dtype="bfloat16", max_tokens=256)
    p = prompts("A", [40])[0]
    s = eng.open()
    want = eng.step([StepEntry(s, p, [len(p) - 1])]).cpu()
    eng.close(s)
    s = eng.open()
    got, prof = eng.profile_step([StepEntry(s, p, [len(p) - 1])])
    eng.close(s)
    assert torch.equal(got.cpu(), want)
    kinds = {w for w, _n, _us in prof.rows()}
    assert {"embed_gather", "add_rmsnorm", "rope_kvwrite", "route_small"} <= kinds and all(us >= 0 for _w, _n, us in prof.rows())
    assert eng.use_graphs and eng.rt.side_stream is not None
    rc = main(["generate", "--model", str(folders["A"]), "--dtype", "float32", "--prompt-ids", ",".join(map(str, p[:6])),
               "--max-tokens", "3", "--profile"])
    out = capsys.readouterr()
    assert rc == 0 and "one decode step, by kernel" in out.err and "gemm_simt" in out.err
