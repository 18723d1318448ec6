"""One layer at sizes near the large models' (7 query heads per key/value head, head 128, a width that is
no power of two, top-8 of 8 experts, a shared expert too wide for the weight-streaming kernel's staging):
the kernels that the tiny models never reach, through the engine, against the plain implementation."""
import numpy as np
import pytest

from gpu_util import Recorder, check_against_plain, engine_for, run_steps, steps_tail, steps_whole
from tiny import random_ids

pytestmark = pytest.mark.gpu

MEDIUM = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": 1, "hidden_size": 1792, "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "intermediate_size": 512, "num_experts": 8, "num_experts_per_tok": 8, "norm_topk_prob": False,
    "moe_intermediate_size": 1280, "shared_expert_intermediate_size": 14336, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": None, "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from esp_b200.config import config_from_dict
    from esp_b200.weights import InitSpec, write_model_folder
    path = tmp_path_factory.mktemp("medium") / "model"
    write_model_folder(config_from_dict(MEDIUM), 77, path, "bfloat16", InitSpec(0.02, 0.02, 0.0))
    return path


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_medium_layer_whole_and_tail(folder, dtype):
    eng = engine_for(folder, dtype, max_tokens=2048)
    rng = np.random.default_rng(5)
    reqs = {"a": random_ids(rng, 300, 1000), "b": random_ids(rng, 70, 1000)}
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps_whole(reqs), rec)
    check_against_plain(folder, dtype, reqs, rec, "medium, whole")
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, steps_tail({"b": reqs["b"]}, 8), rec)
    check_against_plain(folder, dtype, {"b": reqs["b"]}, rec, "medium, last 8 one by one")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_medium_layer_batched_prefill_equals_prefill_alone(folder, dtype):
    """Six prompts of unequal length in one step (thousands of (token, expert) rows: several tiles per
    expert in the grouped products) against the same prompts one at a time."""
    from esp_b200.engine import StepEntry
    eng = engine_for(folder, dtype, max_tokens=4096)
    eng.rt.record_routing = False
    try:
        rng = np.random.default_rng(9)
        prompts = [random_ids(rng, n, 1000) for n in (700, 64, 333, 1, 129, 450)]
        slots = [eng.open() for _ in prompts]
        together = eng.step([StepEntry(s, p, [len(p) - 1, 0]) for s, p in zip(slots, prompts)]).float().cpu().numpy()
        for s in slots:
            eng.close(s)
        for i, p in enumerate(prompts):
            s = eng.open()
            alone = eng.step([StepEntry(s, p, [len(p) - 1, 0])]).float().cpu().numpy()
            eng.close(s)
            got = together[2 * i:2 * i + 2]
            if dtype == "float32":
                assert np.array_equal(got, alone), f"prompt {i}"
            else:
                scale = np.abs(alone).max()
                assert np.abs(got - alone).max() <= 4 * 2.0 ** -8 * scale, f"prompt {i}"
        assert eng.read_status() == 0
    finally:
        eng.rt.record_routing = True


# ---------------------------------------------------------------------------------------------------
# Several layers at head sizes 128 and 64, so that the whole matrix of cuttings runs on the kernels that
# generation uses at the large models' sizes: split-key decode attention, the tensor-memory prefill
# attention (with more (tile, head) items than SMs), the grouped tensor-memory products and the grouped
# weight-streaming product, two cache groups (all keys / a window whose pages are given back), a dense
# layer among sparse ones, a tied head.
# ---------------------------------------------------------------------------------------------------
MEDIUM_B = {
    "hd128": {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
        "num_hidden_layers": 3, "hidden_size": 512, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128,
        "vocab_size": 2000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 3072,
        "intermediate_size": 768, "num_experts": 8, "num_experts_per_tok": 2, "norm_topk_prob": False,
        "moe_intermediate_size": 256, "shared_expert_intermediate_size": 512, "decoder_sparse_step": 1,
        "mlp_only_layers": [1], "use_sliding_window": True, "sliding_window": 200, "max_window_layers": 1,
        "tie_word_embeddings": True,
    },
    "hd64": {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
        "num_hidden_layers": 4, "hidden_size": 384, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 64,
        "vocab_size": 1500, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 1024,
        "intermediate_size": 640, "num_experts": 6, "num_experts_per_tok": 3, "norm_topk_prob": True,
        "moe_intermediate_size": 192, "shared_expert_intermediate_size": 320, "decoder_sparse_step": 2,
        "mlp_only_layers": [], "use_sliding_window": True, "sliding_window": 100, "max_window_layers": 0,
        "tie_word_embeddings": False,
    },
}
# request lengths; the first one gives the tensor-memory attention 20 tiles x 8 heads = 160 items (hd128)
LENGTHS_B = {"hd128": [2500, 150, 420, 65, 300, 33], "hd64": [600, 150, 420, 65, 700, 33]}
# tokens that each request decodes one by one in the batched cutting (the rest is its prompt)
DECODED_B = [32, 5, 40, 32, 1, 0]


@pytest.fixture(scope="module")
def folders_b(tmp_path_factory):
    from esp_b200.config import config_from_dict
    from esp_b200.weights import InitSpec, write_model_folder
    out = {}
    for name, raw in MEDIUM_B.items():
        # "<name>_all": the same model with every expert chosen for every token, for runs in which the engine's
        # expert choices cannot be recorded (decode steps replayed from graphs): in bfloat16 a choice between
        # two nearly equal probabilities may fall either way, and with it every later row of the request
        for variant, change in ((name, {}), (name + "_all", {"num_experts_per_tok": raw["num_experts"]})):
            path = tmp_path_factory.mktemp("medium_b") / variant
            write_model_folder(config_from_dict({**raw, **change}), 91, path, "bfloat16", InitSpec(0.03, 0.02, 0.01))
            out[variant] = path
    return out


def requests_b(name, seed=0):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_ids(rng, n, MEDIUM_B[name]["vocab_size"]) for i, n in enumerate(LENGTHS_B[name])}


def cache_for_one_batch(name):
    """Tokens of cache that hold the larger of the two batches and nothing more."""
    n = LENGTHS_B[name]
    pages = lambda ids: sum((n[i] + 63) // 64 for i in ids)
    return 64 * max(pages([0, 1, 5]), pages([2, 3, 4]))


def cuttings_b(name, reqs):
    from gpu_util import steps_batches
    prompt_lens = {rid: max(1, len(t) - d) for (rid, t), d in zip(reqs.items(), DECODED_B)}
    return {"whole": steps_whole(reqs), "last 32 one by one": steps_tail(reqs, 32),
            "unequal batches": steps_batches(reqs, [["r0", "r1", "r5"], ["r2", "r3", "r4"]], prompt_lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["hd128", "hd64"])
@pytest.mark.parametrize("cutting", ["whole", "last 32 one by one", "unequal batches"])
def test_medium_models_against_plain_in_every_cutting(folders_b, name, dtype, cutting):
    """Every request's logits at every position against the plain implementation.  The batched cutting runs
    two batches one after the other in a cache that holds one, so the second batch lives in the slots and
    pages (of both cache groups) that the first gave back."""
    eng = engine_for(folders_b[name], dtype, max_tokens=cache_for_one_batch(name))
    reqs = requests_b(name)
    rec = Recorder(eng.plan.vocab)
    run_steps(eng, cuttings_b(name, reqs)[cutting], rec)
    check_against_plain(folders_b[name], dtype, reqs, rec, f"medium {name}, {cutting}")
    assert eng.cache.book.slots.available == eng.max_slots
    assert all(g.pool.available == g.pool.n for g in eng.cache.book.groups), "a page was not given back"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["hd128", "hd64"])
def test_medium_models_cuttings_agree_with_decode_steps_replayed_from_graphs(folders_b, name, dtype):
    """The three cuttings against each other with nothing recorded, so that decode steps are captured and
    replayed: bit for bit in float32; in bfloat16 within rounding (rows of a prompt and rows decoded one by
    one go through different kernels, which add in different orders)."""
    folder = folders_b[name if dtype == "float32" else name + "_all"]
    eng = engine_for(folder, dtype, max_tokens=cache_for_one_batch(name), record_routing=False)
    reqs = requests_b(name, seed=4)
    replays = eng.graph_replays
    recs = {}
    for what, steps in cuttings_b(name, reqs).items():
        recs[what] = Recorder(eng.plan.vocab)
        run_steps(eng, steps, recs[what])
    assert eng.graph_replays > replays + 20, "decode steps were meant to replay captured graphs"
    for rid, toks in reqs.items():
        a = recs["whole"].logits_of(rid, range(len(toks)))
        for what in ("last 32 one by one", "unequal batches"):
            b = recs[what].logits_of(rid, range(len(toks)))
            if dtype == "float32":
                assert np.array_equal(a, b), f"{name}, {rid}: whole and {what} differ"
            else:
                assert np.abs(a - b).max() <= 4 * 2.0 ** -8 * np.abs(a).max(), f"{name}, {rid}: whole and {what}"
    if dtype == "bfloat16":
        for what, rec in recs.items():
            check_against_plain(folder, dtype, reqs, rec, f"medium {name}, all experts, graphs, {what}")


@pytest.mark.parametrize("name", ["hd128", "hd64"])
def test_the_same_steps_twice_give_the_same_bits_in_bfloat16(folders_b, name):
    """Nothing in a step depends on the order in which blocks happen to run (the permutation places an expert's
    rows with atomics, the attention's last block combines, the shared expert runs on a second stream): the
    same batches run twice, eagerly and from captured graphs, give identical logits."""
    eng = engine_for(folders_b[name], "bfloat16", max_tokens=cache_for_one_batch(name), record_routing=False)
    reqs = requests_b(name, seed=6)
    steps = cuttings_b(name, reqs)["unequal batches"]
    runs = []
    for _ in range(3):
        rec = Recorder(eng.plan.vocab)
        run_steps(eng, steps, rec)
        runs.append(rec)
    for rid, toks in reqs.items():
        first = runs[0].logits_of(rid, range(len(toks)))
        for other in runs[1:]:
            assert np.array_equal(first, other.logits_of(rid, range(len(toks)))), f"{name}, {rid}: two runs differ"


def test_window_pages_are_trimmed_and_reused_at_head_size_64(folders_b):
    """All layers windowed (100 keys): a prompt longer than two pages, a second portion after the window has
    passed whole pages, single tokens across positions 256 and 512, then another request in a cache so small
    that it can only live in the pages the window gave back."""
    from esp_b200.engine import StepEntry
    name, dtype = "hd64", "bfloat16"
    eng = engine_for(folders_b[name], dtype, max_tokens=6 * 64)
    rng = np.random.default_rng(12)
    a, b = random_ids(rng, 530, 1500), random_ids(rng, 330, 1500)
    rec = Recorder(eng.plan.vocab)
    steps = [([("a", a[:140], list(range(140)))], []), ([("a", a[140:250], list(range(110)))], [])]
    steps += [([("a", [a[i]], [0])], []) for i in range(250, 262)]
    steps += [([("a", a[262:505], list(range(243)))], [])]
    steps += [([("a", [a[i]], [0])], []) for i in range(505, 520)]
    # b starts while a still lives (a holds three pages of the six), then a ends and b's prompt takes five
    steps += [([("a", [a[520]], [0]), ("b", b[:1], [0])], [])]
    steps += [([("a", a[521:], list(range(9)))], ["a"])]
    steps += [([("b", b[1:300], list(range(299)))], [])]
    steps += [([("b", [b[i]], [0])], ["b"] if i == 329 else []) for i in range(300, 330)]
    run_steps(eng, steps, rec)
    check_against_plain(folders_b[name], dtype, {"a": a, "b": b}, rec, "windowed pages")
    (group,) = eng.cache.book.groups
    assert group.layout.window == 100 and group.pool.available == group.pool.n == 6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [37, 2])
def test_feed_forward_rows_cut_into_portions_change_nothing(folders_b, dtype, chunk):
    """The feed-forward parts cut a step's rows into portions above a limit that no model reaches in tests;
    with the limit at 37 and at 2 rows (a last portion of one row, a row count of portions * k + 1) the
    logits are the uncut ones: bit for bit in float32, within rounding in bfloat16."""
    from esp_b200.engine import StepEntry
    eng = engine_for(folders_b["hd128"], dtype, max_tokens=1024, record_routing=False)
    rng = np.random.default_rng(13)
    toks = random_ids(rng, 2 * 37 + 1, 2000)
    want = list(range(len(toks)))

    def run():
        s = eng.open()
        out = eng.step([StepEntry(s, toks, want)]).float().cpu().numpy()
        tail = eng.step([StepEntry(s, toks[:3], [0, 1, 2])]).float().cpu().numpy()
        eng.close(s)
        return np.concatenate([out, tail])

    uncut = run()
    limit = eng.rt.ffn_chunk_tokens
    eng.rt.ffn_chunk_tokens = chunk
    try:
        cut = run()
    finally:
        eng.rt.ffn_chunk_tokens = limit
    assert eng.read_status() == 0
    if dtype == "float32":
        assert np.array_equal(cut, uncut)
    else:
        assert np.abs(cut - uncut).max() <= 4 * 2.0 ** -8 * np.abs(uncut).max()


def test_shared_expert_ahead_of_the_router_changes_nothing(folders_b):
    """Steps of many rows start the shared expert's first product on a second stream, on fewer SMs, before the
    router runs.  A prompt of 1,700 tokens through that path (whole, and cut into portions of 800 rows so that
    two portions take it and a last one of 100 rows does not) gives the logits of the same prompt with the
    second stream never used: rows do not depend on where their product ran."""
    from esp_b200.engine import StepEntry
    from esp_b200.parts import ffn
    eng = engine_for(folders_b["hd128"], "bfloat16", max_tokens=2048, record_routing=False)
    rng = np.random.default_rng(17)
    toks = random_ids(rng, 1700, 2000)
    want = [0, 1, 767, 768, 799, 800, 1599, 1600, 1699]

    def run():
        s = eng.open()
        out = eng.step([StepEntry(s, toks, want)]).float().cpu().numpy()
        eng.close(s)
        return out

    assert len(toks) >= ffn.AHEAD_ROWS
    ahead = run()
    limit, rows = eng.rt.ffn_chunk_tokens, ffn.AHEAD_ROWS
    try:
        eng.rt.ffn_chunk_tokens = 800
        portions = run()
        ffn.AHEAD_ROWS = 10 ** 9
        eng.rt.ffn_chunk_tokens = limit
        in_line = run()
    finally:
        eng.rt.ffn_chunk_tokens, ffn.AHEAD_ROWS = limit, rows
    assert eng.read_status() == 0
    assert np.array_equal(ahead, in_line)
    assert np.abs(portions - in_line).max() <= 4 * 2.0 ** -8 * np.abs(in_line).max()


def test_a_single_token_step_reads_exactly_top_k_experts_per_sparse_layer(folders_b):
    """The engine's counters: a step of one token touches exactly k experts in every sparse layer
    (crates/esp/src/infer/decoder/architecture_tests.rs:220-236); a step of several tokens touches at most
    k per token and at least k."""
    from esp_b200.engine import StepEntry
    for name, dtype in (("hd128", "bfloat16"), ("hd64", "float32")):
        raw = MEDIUM_B[name]
        sparse = sum((i + 1) % raw["decoder_sparse_step"] == 0 and i not in raw["mlp_only_layers"]
                     for i in range(raw["num_hidden_layers"]))
        k = raw["num_experts_per_tok"]
        eng = engine_for(folders_b[name], dtype, max_tokens=1024, record_routing=False)
        s = eng.open()
        before = eng.counters()
        eng.step([StepEntry(s, [5, 6, 7, 8, 9], [])])
        mid = eng.counters()
        assert k * sparse <= mid["expert_reads"] - before["expert_reads"] <= min(5 * k, raw["num_experts"]) * sparse
        assert mid["tokens"] - before["tokens"] == 5 and mid["steps"] - before["steps"] == 1
        for t in range(6):                      # eager, captured and replayed decode steps all count
            was = eng.counters()
            eng.step([StepEntry(s, [t], [0])])
            now = eng.counters()
            assert now["expert_reads"] - was["expert_reads"] == k * sparse, f"{name}: decode step {t}"
            assert now["kv_bytes_read"] > was["kv_bytes_read"]
        eng.close(s)
