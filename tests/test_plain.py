"""The plain implementation against the outputs that the reference project
records for its two Qwen2-MoE checkpoints (tests/golden/README.md)."""
import json
from pathlib import Path

import numpy as np
import pytest

import plain_qwen2_moe as plain

GOLDEN = Path(__file__).parent / "golden"
CASES = {c["name"]: c for c in json.loads((GOLDEN / "recorded_outputs.json").read_text())["cases"]}


@pytest.mark.parametrize("name", ["qwen2_moe", "qwen2_moe_normalized"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_recorded_logits_and_greedy_ids(name, dtype):
    case = CASES[name]
    c, w = plain.load_model(GOLDEN / name)
    logits = plain.forward_logits(c, w, case["input_ids"], dtype)
    err = np.abs(logits[-1] - np.asarray(case["last_logits"], dtype=np.float32)).max()
    # the reference's own acceptance is 2e-5 (architecture_tests.rs:237-247)
    assert err < (2e-6 if dtype is np.float32 else 5e-7), err
    ids = plain.generate(c, w, case["input_ids"], len(case["generated_ids"]), dtype=dtype)
    assert ids == case["generated_ids"]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_recorded_outputs_of_the_windowed_checkpoint_pin_the_mask(dtype):
    """The reference's dense ``qwen2`` checkpoint runs the same attention code with q/k/v bias, one key/value
    head for two query heads, ``layer_types`` [full, sliding] and a window of 3 over a prompt of 9 tokens:
    its recorded logits pin the window's mask (a query sees itself and two predecessors), which layer is
    windowed, and the decode steps behind the window.  Every layer is dense here."""
    case = CASES["qwen2"]
    c, w = plain.load_model(GOLDEN / "qwen2")
    assert [plain.layer_window(c, i) for i in range(2)] == [None, 3]
    logits = plain.forward_logits(c, w, case["input_ids"], dtype)
    err = np.abs(logits[-1] - np.asarray(case["last_logits"], dtype=np.float32)).max()
    assert err < (2e-6 if dtype is np.float32 else 5e-7), err
    assert plain.generate(c, w, case["input_ids"], 4, dtype=dtype) == case["generated_ids"]
    # the recorded numbers do depend on the window: with one key more or one key fewer they are missed
    for other in (2, 4, None):
        wrong = dict(c, sliding_window=other) if other else dict(c, layer_types=None, use_sliding_window=False)
        off = np.abs(plain.forward_logits(wrong, w, case["input_ids"], dtype)[-1] - np.asarray(case["last_logits"])).max()
        assert off > 1e-4, (other, off)
    # without layer_types, use_sliding_window + max_window_layers 1 name the same layer
    assert [plain.layer_window(dict(c, layer_types=None), i) for i in range(2)] == [None, 3]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_recorded_outputs_of_a_checkpoint_whose_head_size_is_not_width_over_heads(dtype):
    """The reference's dense ``mistral`` checkpoint runs the same attention code with ``head_dim`` 12 at a
    width of 16 with 2 heads (so that q is 24 wide and the scores are divided by sqrt(12)), one key/value head
    for two query heads and a window of 3 on every layer.  Its recorded logits pin the explicit head size;
    every layer is dense here and no projection has a bias."""
    case = CASES["mistral"]
    c, w = plain.load_model(GOLDEN / "mistral")
    assert c["head_dim"] == 12 and c["hidden_size"] // c["num_attention_heads"] == 8
    assert [plain.layer_window(c, i) for i in range(2)] == [3, 3]
    logits = plain.forward_logits(c, w, case["input_ids"], dtype)
    err = np.abs(logits[-1] - np.asarray(case["last_logits"], dtype=np.float32)).max()
    assert err < (2e-6 if dtype is np.float32 else 5e-7), err
    assert plain.generate(c, w, case["input_ids"], 4, dtype=dtype) == case["generated_ids"]
    # the numbers do depend on the divisor: with sqrt(width / heads) they are missed
    import unittest.mock as mock
    real_sqrt = np.sqrt
    wrong = dict(c)
    off = None
    with mock.patch.object(plain.np, "sqrt", lambda v, *a, **k: real_sqrt(8.0 if np.ndim(v) == 0 and float(v) == 12.0 else v, *a, **k)):
        off = np.abs(plain.forward_logits(wrong, w, case["input_ids"], dtype)[-1] - np.asarray(case["last_logits"])).max()
    assert off > 1e-5, off


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_recorded_outputs_of_a_plain_dense_checkpoint(dtype):
    """The reference's dense ``llama`` checkpoint: the same attention and feed-forward code with no bias, no
    window, one key/value head for two query heads and a head size equal to width / heads.  With the ``qwen2`` and
    ``mistral`` cases it shows that neither the window nor the explicit head size leaks into the case without them."""
    case = CASES["llama"]
    c, w = plain.load_model(GOLDEN / "llama")
    assert [plain.layer_window(c, i) for i in range(2)] == [None, None]
    assert not any(name.endswith("_proj.bias") for name in w)
    logits = plain.forward_logits(c, w, case["input_ids"], dtype)
    err = np.abs(logits[-1] - np.asarray(case["last_logits"], dtype=np.float32)).max()
    assert err < (2e-6 if dtype is np.float32 else 5e-7), err
    assert plain.generate(c, w, case["input_ids"], len(case["generated_ids"]), dtype=dtype) == case["generated_ids"]


def test_splitmix64_known_values():
    # first outputs of splitmix64 from seed 0 (public test vector of the generator)
    r = plain.SplitMix64(0)
    assert r.next_u64() == 0xE220A8397B1DCDAF
    assert r.next_u64() == 0x6E789E6AA1B965F4
    a = plain.SplitMix64(7)
    b = plain.SplitMix64(7)
    for _ in range(5):
        a.next_u64()
    b.skip(5)
    assert a.next_u64() == b.next_u64()


def test_sampler_low_temperature_is_greedy_and_top_p_small_is_argmax():
    rng = np.random.default_rng(0)
    row = rng.normal(size=50).astype(np.float32)
    assert plain.sample_row(row, 1e-4, None, plain.SplitMix64(1)) == int(np.argmax(row))
    assert plain.sample_row(row, 1.0, 1e-6, plain.SplitMix64(2)) == int(np.argmax(row))


def test_window_masks_far_keys():
    c, w = plain.load_model(GOLDEN / "qwen2_moe")
    x = np.random.default_rng(0).normal(size=(12, c["hidden_size"])).astype(np.float32)
    full = plain.attention(c, w, "model.layers.0.self_attn.", x, None)
    win = plain.attention(c, w, "model.layers.0.self_attn.", x, 4)
    assert np.allclose(full[:4], win[:4], atol=1e-6)
    assert not np.allclose(full[8:], win[8:], atol=1e-6)
    # a query sees itself and window-1 predecessors: changing token 0 leaves row 4 unchanged
    x2 = x.copy(); x2[0] += 1.0
    win2 = plain.attention(c, w, "model.layers.0.self_attn.", x2, 4)
    assert np.allclose(win[4:], win2[4:], atol=1e-6)
    assert not np.allclose(win[3], win2[3], atol=1e-6)
