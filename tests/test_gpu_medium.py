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
