"""Weights: the safetensors reader and writer, binding by name, the one error
that lists everything wrong, and random model folders
(cases follow crates/esp/src/infer/decoder/loader.rs:686-825)."""
import json
import struct

import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from esp_b200.config import config_from_dict
from esp_b200.errors import InvalidWeights
from esp_b200.weights import (FolderSource, InitSpec, RandomSource, check_names_and_shapes, open_model_folder,
                              parameter_specs, read_tensor, write_model_folder, write_safetensors)
from esp_b200.weights.random_init import normal_values, tensor_key
from tiny import TINY_A, TINY_B, make_folder


def test_round_trip_all_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    write_safetensors(tmp_path / "model.safetensors", t)
    metas = open_model_folder(tmp_path)
    for k, v in t.items():
        got = read_tensor(metas[k])
        assert got.dtype == v.dtype and torch.equal(got, v)


def test_own_reader_agrees_with_the_plain_reader(tmp_path):
    folder = make_folder(tmp_path, "A", store="bfloat16")
    metas = open_model_folder(folder)
    w = plain.read_safetensors(folder / "model.safetensors")
    assert set(metas) == set(w)
    for name in list(metas)[:10]:
        assert np.array_equal(read_tensor(metas[name]).float().numpy(), w[name])


def test_parameter_names_are_the_checkpoint_names():
    names = {s.name for s in parameter_specs(config_from_dict(TINY_B))}
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names
    assert "model.layers.0.mlp.gate_proj.weight" in names            # layer 0 is dense
    assert "model.layers.1.mlp.experts.5.down_proj.weight" in names  # layer 1 is sparse
    assert "model.layers.1.mlp.shared_expert_gate.weight" in names
    assert "model.layers.2.self_attn.q_proj.bias" in names
    assert "model.layers.2.self_attn.o_proj.bias" not in names
    assert not any("layers.0.mlp.experts" in n for n in names)


def _specs_and_source(tmp_path, case="A", mutate=None):
    folder = make_folder(tmp_path, case, store="float32")
    cfg = config_from_dict(TINY_A if case == "A" else TINY_B)
    if mutate is not None:
        metas = open_model_folder(folder)
        tensors = {n: read_tensor(m) for n, m in metas.items()}
        mutate(tensors)
        write_safetensors(folder / "model.safetensors", tensors)
    return parameter_specs(cfg), FolderSource(folder), cfg


def test_good_checkpoint_passes(tmp_path):
    specs, src, cfg = _specs_and_source(tmp_path)
    check_names_and_shapes(specs, src, cfg.plan().tolerated_suffixes)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    def mutate(t):
        del t["model.layers.0.self_attn.q_proj.bias"]
        del t["model.layers.1.mlp.experts.3.up_proj.weight"]
        t["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(64)
        t["model.layers.7.input_layernorm.weight"] = torch.zeros(64)
        t["model.norm.weight"] = torch.zeros(65)
        t["model.layers.0.mlp.gate.weight"] = torch.zeros(4, 32)
    specs, src, cfg = _specs_and_source(tmp_path, mutate=mutate)
    with pytest.raises(InvalidWeights) as e:
        check_names_and_shapes(specs, src, cfg.plan().tolerated_suffixes)
    msg = str(e.value)
    for needle in ("missing tensors (2)", "q_proj.bias", "experts.3.up_proj.weight", "unexpected tensors",
                   "o_proj.bias", "layers.7.input_layernorm", "wrong shapes (2)", "model.norm.weight: stored [65]",
                   "expected [64]", "mlp.gate.weight: stored [4, 32]"):
        assert needle in msg, (needle, msg)


def test_inv_freq_is_tolerated_and_head_rules(tmp_path):
    def add_inv_freq(t):
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    specs, src, cfg = _specs_and_source(tmp_path, mutate=add_inv_freq)
    check_names_and_shapes(specs, src, cfg.plan().tolerated_suffixes)

    def drop_head(t):
        del t["lm_head.weight"]
    specs, src, cfg = _specs_and_source(tmp_path, mutate=drop_head)
    with pytest.raises(InvalidWeights, match="lm_head.weight"):
        check_names_and_shapes(specs, src, cfg.plan().tolerated_suffixes)
    # a tied model needs no head, and may carry one
    specs_b, src_b, cfg_b = _specs_and_source(tmp_path, "B")
    assert "lm_head.weight" not in src_b.names()
    check_names_and_shapes(specs_b, src_b, cfg_b.plan().tolerated_suffixes)
    specs_b, src_b, cfg_b = _specs_and_source(tmp_path, "B", mutate=lambda t: t.update(
        {"lm_head.weight": torch.zeros(384, 96)}))
    check_names_and_shapes(specs_b, src_b, cfg_b.plan().tolerated_suffixes)


def test_integer_weight_is_refused(tmp_path):
    specs, src, cfg = _specs_and_source(tmp_path, mutate=lambda t: t.update(
        {"model.norm.weight": torch.ones(64, dtype=torch.int32)}))
    with pytest.raises(InvalidWeights, match="not floating point"):
        check_names_and_shapes(specs, src, ())


@pytest.mark.parametrize("damage", ["short", "header_len", "not_json", "bad_dtype", "bad_offsets", "gap"])
def test_malformed_files(tmp_path, damage):
    good = {"x": torch.zeros(4), "y": torch.ones(2)}
    path = tmp_path / "model.safetensors"
    write_safetensors(path, good)
    blob = path.read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    if damage == "short":
        path.write_bytes(blob[:5])
    elif damage == "header_len":
        path.write_bytes(struct.pack("<Q", 1 << 40) + blob[8:])
    elif damage == "not_json":
        path.write_bytes(blob[:8] + b"{" * hlen + blob[8 + hlen:])
    else:
        if damage == "bad_dtype":
            header["x"]["dtype"] = "F8_E4M3"
        elif damage == "bad_offsets":
            header["x"]["data_offsets"] = [0, 12]
        elif damage == "gap":
            header["y"]["data_offsets"] = [20, 28]
        h = json.dumps(header).encode()
        path.write_bytes(struct.pack("<Q", len(h)) + h + blob[8 + hlen:] + b"\0" * 16)
    with pytest.raises(InvalidWeights):
        open_model_folder(tmp_path)


def test_sharded_folder(tmp_path):
    write_safetensors(tmp_path / "s1.safetensors", {"a": torch.zeros(2)})
    write_safetensors(tmp_path / "s2.safetensors", {"b": torch.ones(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    metas = open_model_folder(tmp_path)
    assert set(metas) == {"a", "b"} and torch.equal(read_tensor(metas["b"]), torch.ones(3))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s1.safetensors"}}))
    with pytest.raises(InvalidWeights):
        open_model_folder(tmp_path)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../s1.safetensors"}}))
    with pytest.raises(InvalidWeights):
        open_model_folder(tmp_path)


def test_random_folder_is_reproducible_and_follows_the_init(tmp_path):
    a1 = make_folder(tmp_path / "1", "A", seed=5)
    a2 = make_folder(tmp_path / "2", "A", seed=5)
    a3 = make_folder(tmp_path / "3", "A", seed=6)
    assert (a1 / "model.safetensors").read_bytes() == (a2 / "model.safetensors").read_bytes()
    assert (a1 / "model.safetensors").read_bytes() != (a3 / "model.safetensors").read_bytes()
    c, w = plain.load_model(a1)
    emb = w["model.embed_tokens.weight"]
    assert abs(emb.std() - 0.02) < 0.002 and abs(emb.mean()) < 0.002
    assert abs(w["model.layers.0.self_attn.q_proj.bias"].std() - 0.02) < 0.008
    g = w["model.layers.1.input_layernorm.weight"]
    assert abs(g.mean() - 1.0) < 0.01 and 0.002 < g.std() < 0.03
    cb, wb = plain.load_model(make_folder(tmp_path, "B"))
    assert np.all(wb["model.layers.0.self_attn.k_proj.bias"] == 0) and np.all(wb["model.norm.weight"] == 1)
    assert abs(wb["model.layers.1.mlp.experts.2.up_proj.weight"].std() - 0.05) < 0.005
    assert json.loads((a1 / "config.json").read_text())["architectures"] == ["Qwen2MoeForCausalLM"]


def test_values_depend_on_name_and_index_only():
    k = tensor_key(3, "model.norm.weight")
    whole = normal_values(k, 1000, 0.0, 1.0)
    assert np.array_equal(whole[:10], normal_values(k, 10, 0.0, 1.0))
    assert tensor_key(3, "a") != tensor_key(3, "b") and tensor_key(3, "a") != tensor_key(4, "a")
    assert abs(whole.mean()) < 0.15 and abs(whole.std() - 1.0) < 0.1
