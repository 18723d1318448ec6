"""The layer sizes of Qwen1.5-MoE-A2.7B (width 2048, 16 heads of 128, vocabulary 151,936, 60 experts of
1,408, top-4, shared expert of 5,632) with 2 of its 24 layers, so that it fits a test: the three cuttings
agree (bit for bit in float32), and the logits agree with the plain implementation, which is given the very
weights the engine holds (random, made on the device, read back)."""
import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from gpu_util import Recorder, check_against_plain, run_steps, steps_batches, steps_tail, steps_whole
from tiny import random_ids

pytestmark = pytest.mark.gpu

LAYERS, LAYERS_OF_MODEL = 2, 24
A27B_2L = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": LAYERS, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "intermediate_size": 5632, "num_experts": 60, "num_experts_per_tok": 4,
    "norm_topk_prob": False, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": None,
    "tie_word_embeddings": False,
}
# The second shape of the reference's real-model gates, Qwen2-57B-A14B, with 1 of its 28 layers: 7 query heads per
# key/value head, top-8 of 64 experts, a shared expert whose down-projection has rows of 20,480 values (more than the
# weight-streaming kernel stages at once).
Q57B_1L = dict(A27B_2L, num_hidden_layers=1, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               max_position_embeddings=32768, intermediate_size=18944, num_experts=64, num_experts_per_tok=8,
               moe_intermediate_size=2560, shared_expert_intermediate_size=20480)
SHAPES = {"a2.7b": (A27B_2L, f"A2.7B sizes, {LAYERS} of {LAYERS_OF_MODEL} layers"), "57b-a14b": (Q57B_1L, "57B-A14B sizes, 1 of 28 layers")}
LENGTHS = [200, 37, 131, 256, 9, 64]
DECODED = [8, 8, 8, 8, 8, 0]


class Keeping:
    """A weight source that remembers where each tensor went, so that the test can read the model's
    weights back exactly as the engine holds them."""

    def __init__(self, inner, views):
        self.inner, self.views = inner, views

    def names(self):
        return self.inner.names()

    def dtype(self, name):
        return self.inner.dtype(name)

    def shape(self, name):
        return self.inner.shape(name)

    def read_into(self, name, view):
        self.inner.read_into(name, view)
        self.views[name] = view


def make_engine(shape, dtype, views=None):
    from esp_b200.config import config_from_dict
    from esp_b200.engine import Engine
    from esp_b200.weights import InitSpec, RandomSource
    views = {} if views is None else views
    factory = lambda specs: Keeping(RandomSource(specs, 5, InitSpec(0.02, 0.02, 0.0), torch.bfloat16), views)
    eng = Engine(config_from_dict(SHAPES[shape][0]), factory, dtype=dtype, max_tokens=1024, max_slots=8)
    eng.rt.record_routing = True
    return eng, views


@pytest.fixture(scope="module", params=["a2.7b", "57b-a14b"])
def model(request):
    """(shape, bfloat16 engine, (config, weights) for the plain implementation: the bfloat16 values the
    engines hold, widened)."""
    eng, views = make_engine(request.param, "bfloat16")
    weights = {name: v.float().cpu().numpy() for name, v in views.items()}
    config = plain.read_config_dict(dict(SHAPES[request.param][0]))
    yield request.param, eng, (config, weights)
    del eng, weights
    torch.cuda.empty_cache()


def requests(seed=0):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_ids(rng, n, A27B_2L["vocab_size"]) for i, n in enumerate(LENGTHS)}


def cuttings(reqs):
    prompt_lens = {rid: max(1, len(t) - d) for (rid, t), d in zip(reqs.items(), DECODED)}
    return {"whole": steps_whole(reqs), "last 8 one by one": steps_tail(reqs, 8),
            "unequal batches": steps_batches(reqs, [["r0", "r1", "r5"], ["r2", "r3", "r4"]], prompt_lens)}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_real_layer_sizes_three_cuttings_and_plain(model, dtype):
    shape, eng_bf16, plain_model = model
    if dtype == "bfloat16":
        eng = eng_bf16
    else:
        eng, _ = make_engine(shape, "float32")      # the same values (stored as bfloat16), widened exactly
    reqs = requests()
    recs = {}
    for what, steps in cuttings(reqs).items():
        recs[what] = Recorder(eng.plan.vocab)
        run_steps(eng, steps, recs[what])
    # every position of the two shortest requests and the last positions of the others
    at = {rid: (range(len(t)) if len(t) <= 40 else range(len(t) - 9, len(t))) for rid, t in reqs.items()}
    for what, rec in recs.items():
        check_against_plain(plain_model, dtype, reqs, rec, f"{SHAPES[shape][1]}, {what}", positions=at)
    # in bfloat16 each cutting is held against the plain implementation with its own expert choices (a choice
    # between nearly equal probabilities may fall differently in two cuttings); in float32 the cuttings
    # must agree bit for bit
    if dtype == "float32":
        for rid, toks in reqs.items():
            a = recs["whole"].logits_of(rid, range(len(toks)))
            for what in ("last 8 one by one", "unequal batches"):
                assert np.array_equal(a, recs[what].logits_of(rid, range(len(toks)))), f"{rid}: whole and {what} differ"
    del eng
    torch.cuda.empty_cache()
