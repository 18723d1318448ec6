"""The engine against the plain implementation on the two tiny models, in
32-bit and in bfloat16: each request alone and whole; the last 32 tokens one
by one; batches of unequal lengths whose shorter requests end earlier, one
batch after another so that slots and pages are used again; long decoding; the
first tokens of a sequence."""
import numpy as np
import pytest
import torch

from esp_b200.engine import Engine
from gpu_util import (Recorder, check_against_plain, engine_for, plain_model, run_steps, steps_batches, steps_tail,
                      steps_whole)
from tiny import CASES, make_folder, random_ids

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [100, 45, 70, 33, 128, 7], "B": [200, 40, 130, 65, 256, 1], "C": [150, 40, 90, 33, 160, 2]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {case: make_folder(tmp, case) for case in CASES}


def requests_for(case, seed=0):
    rng = np.random.default_rng(seed)
    vocab = CASES[case][0]["vocab_size"]
    return {f"r{i}": random_ids(rng, n, vocab) for i, n in enumerate(LENGTHS[case])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_each_request_alone_and_whole(folders, case, dtype):
    eng = engine_for(folders[case], dtype)
    reqs = requests_for(case)
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps_whole(reqs), rec)
    check_against_plain(folders[case], dtype, reqs, rec, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(folders, case, dtype):
    eng = engine_for(folders[case], dtype)
    reqs = requests_for(case)
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps_tail(reqs, 32), rec)
    check_against_plain(folders[case], dtype, reqs, rec, "tail of 32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_unequal_batches_one_after_another(folders, case, dtype):
    # a cache just large enough for one batch, so that the second batch can only
    # run in the slots and pages that the first one gave back
    eng = engine_for(folders[case], dtype, max_tokens={"A": 3 * 128, "B": 3 * 256, "C": 3 * 192}[case])
    reqs = requests_for(case)
    prompt_lens = {rid: max(1, len(t) - d) for (rid, t), d in zip(reqs.items(), [32, 5, 50, 32, 1, 0])}
    batches = [["r0", "r1", "r5"], ["r2", "r3", "r4"]]
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps_batches(reqs, batches, prompt_lens), rec)
    check_against_plain(folders[case], dtype, reqs, rec, "unequal batches")
    assert eng.cache.book.slots.available == eng.max_slots
    assert all(g.pool.available == g.pool.n for g in eng.cache.book.groups)


@pytest.mark.parametrize("case", ["A", "B"])
def test_cuttings_agree_bit_for_bit_in_float32(folders, case):
    eng = engine_for(folders[case], "float32")
    reqs = requests_for(case, seed=3)
    recs = []
    prompt_lens = {rid: max(1, len(t) - d) for (rid, t), d in zip(reqs.items(), [32, 5, 50, 32, 1, 0])}
    for steps in (steps_whole(reqs), steps_tail(reqs, 32),
                  steps_batches(reqs, [["r0", "r1", "r2"], ["r3", "r4", "r5"]], prompt_lens)):
        rec = Recorder(eng.plan.vocab)
        run_steps(eng, steps, rec)
        recs.append(rec)
    for rid, toks in reqs.items():
        a = recs[0].logits_of(rid, range(len(toks)))
        for other in recs[1:]:
            assert np.array_equal(a, other.logits_of(rid, range(len(toks)))), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B"])
def test_long_decoding_and_first_tokens(folders, case, dtype):
    """Three prompt tokens, then one token at a time to the model's last
    position; and sequences of one, two and three tokens."""
    eng = engine_for(folders[case], dtype)
    raw = CASES[case][0]
    rng = np.random.default_rng(7)
    long = random_ids(rng, raw["max_position_embeddings"], raw["vocab_size"])
    reqs = {"long": long}
    steps = [([("long", long[:3], [0, 1, 2])], [])]
    for i in range(3, len(long)):
        steps.append(([("long", [long[i]], [0])], ["long"] if i == len(long) - 1 else []))
    for n in (1, 2, 3):
        reqs[f"s{n}"] = random_ids(rng, n, raw["vocab_size"])
        steps.append(([(f"s{n}", reqs[f"s{n}"], list(range(n)))], [f"s{n}"]))
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps, rec)
    check_against_plain(folders[case], dtype, reqs, rec, "long decoding / first tokens")


def test_step_refuses_what_cannot_run_and_changes_nothing(folders):
    from esp_b200.engine import StepEntry
    from esp_b200.errors import CacheFull, InvalidRequest
    eng = engine_for(folders["A"], "float32", max_tokens=128)
    s = eng.open()
    free = eng.cache.book.groups[0].pool.available
    for bad in ([StepEntry(s, [], [])], [StepEntry(s, [256], [0])], [StepEntry(s, [-1], [0])],
                [StepEntry(s, [1, 2], [2])], [StepEntry(s, [1], [0]), StepEntry(s, [2], [0])],
                [StepEntry(s, [1] * 129, [])], [StepEntry(99, [1], [0])], []):
        with pytest.raises(InvalidRequest):
            eng.step(bad)
    t = eng.open()
    with pytest.raises(CacheFull):
        eng.step([StepEntry(s, [1] * 100, []), StepEntry(t, [1] * 100, [])])
    assert eng.length(s) == 0 and eng.cache.book.groups[0].pool.available == free
    out = eng.step([StepEntry(s, [1, 2, 3], [])])
    assert out.shape == (0, 256) and eng.length(s) == 3
    eng.close(s)
    eng.close(t)
    with pytest.raises(InvalidRequest):
        eng.close(t)


def test_checkpoint_streams_to_the_device_in_chunks_and_refuses_non_finite_values(folders, tmp_path):
    """The loader reads a tensor in chunks through pinned buffers; with chunks of 1,000 bytes (no multiple of an
    element) the model's logits are those of the ordinary load.  A NaN or an infinity anywhere in a tensor is
    found on the device and named."""
    import shutil
    from esp_b200.engine import StepEntry
    from esp_b200.errors import InvalidWeights
    from esp_b200.weights import FolderSource
    from esp_b200.weights.safetensors_io import open_model_folder, read_tensor, write_safetensors
    toks = requests_for("B")["r1"]
    want = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folders["B"], dtype=dtype, max_tokens=256)
        s = eng.open()
        want[dtype] = eng.step([StepEntry(s, toks, [len(toks) - 1])]).cpu()
    chunk = FolderSource.CHUNK_BYTES
    FolderSource.CHUNK_BYTES = 1000
    try:
        for dtype in ("float32", "bfloat16"):
            eng = Engine.from_folder(folders["B"], dtype=dtype, max_tokens=256)
            s = eng.open()
            assert torch.equal(eng.step([StepEntry(s, toks, [len(toks) - 1])]).cpu(), want[dtype])
    finally:
        FolderSource.CHUNK_BYTES = chunk
    # one bad value in the middle of a tensor, one at the very end of another
    bad = tmp_path / "bad"
    shutil.copytree(folders["B"], bad)
    tensors = {n: read_tensor(m) for n, m in open_model_folder(bad).items()}
    tensors["model.layers.1.mlp.experts.2.up_proj.weight"].view(-1)[1234] = float("nan")
    tensors["model.norm.weight"].view(-1)[-1] = float("inf")
    write_safetensors(bad / "model.safetensors", tensors)
    for dtype in ("float32", "bfloat16"):
        with pytest.raises(InvalidWeights) as e:
            Engine.from_folder(bad, dtype=dtype, max_tokens=256)
        assert "experts.2.up_proj" in str(e.value) and "model.norm.weight" in str(e.value) and "not finite" in str(e.value)
