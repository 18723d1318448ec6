"""Configuration: what is accepted, what is refused and what is derived
(the matrix follows crates/esp/src/infer/decoder/config.rs:597-838)."""
import json

import pytest

from esp_b200.config import Qwen2MoeConfig, config_from_dict, config_from_json, supported_architectures
from esp_b200.errors import InvalidConfig, Unsupported
from tiny import TINY_A, TINY_B


def test_registry_names_the_architecture():
    assert "Qwen2MoeForCausalLM" in supported_architectures()
    assert isinstance(config_from_dict(TINY_A), Qwen2MoeConfig)
    only_type = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert isinstance(config_from_dict(only_type), Qwen2MoeConfig)


def test_defaults_match_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in (
        "rms_norm_eps", "rope_theta", "num_key_value_heads", "head_dim", "norm_topk_prob", "decoder_sparse_step",
        "mlp_only_layers", "tie_word_embeddings")}
    c = config_from_dict(raw)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.kv_heads == c.num_attention_heads and c.resolved_head_dim == 16
    assert c.norm_topk_prob is False and c.decoder_sparse_step == 1 and c.mlp_only_layers == []
    assert c.tie_word_embeddings is False


def test_derived_layer_kinds_and_windows():
    b = config_from_dict(TINY_B)
    assert [b.layer_is_moe(i) for i in range(3)] == [False, True, False]
    assert [b.layer_window(i) for i in range(3)] == [None, 16, 16]
    a = config_from_dict(TINY_A)
    assert all(a.layer_is_moe(i) for i in range(2)) and a.layer_window(1) is None
    # max_window_layers defaults to 28: windowing starts at layer 28
    c = config_from_dict({**TINY_B, "max_window_layers": None})
    assert [c.layer_window(i) for i in range(3)] == [None, None, None]
    # use_sliding_window absent: no window either
    d = config_from_dict({k: v for k, v in TINY_B.items() if k != "use_sliding_window"})
    assert d.layer_window(2) is None
    e = config_from_dict({**TINY_B, "layer_types": ["full_attention", "sliding_attention", "full_attention"]})
    assert [e.layer_window(i) for i in range(3)] == [None, 16, None]


def test_bias_rules_ignore_the_bias_keys():
    c = config_from_dict({**TINY_A, "attention_bias": False, "qkv_bias": False})
    assert c.qkv_bias is True and c.output_bias is False
    plan = c.plan()
    assert plan.blocks[0].mixer.qkv_bias and not plan.blocks[0].mixer.out_bias


def test_plan_carries_every_size_from_the_config():
    plan = config_from_dict(TINY_B).plan()
    assert plan.hidden == 96 and plan.vocab == 384 and plan.head_weight is None
    m = plan.blocks[1].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.window) == (4, 1, 24, 16)
    assert m.position.theta == 1000000.0 and m.position.max_positions == 256
    f = plan.blocks[1].ffn
    assert (f.num_experts, f.top_k, f.norm_topk, f.expert_intermediate, f.shared_intermediate) == (6, 3, True, 48, 80)
    assert plan.blocks[0].ffn.kind == "swiglu" and plan.blocks[0].ffn.intermediate == 128
    assert plan.blocks[0].mixer_norm.eps == 1e-5
    assert [e.layer for e in plan.schedule] == [0, 1, 2]


def test_eos_forms():
    assert config_from_dict({**TINY_A, "eos_token_id": 7}).stop_token_ids() == (7,)
    assert config_from_dict({**TINY_A, "eos_token_id": [7, 9]}).stop_token_ids() == (7, 9)
    assert config_from_dict(TINY_A).stop_token_ids() == ()


@pytest.mark.parametrize("patch, feature", [
    ({"text_config": {}}, "text_config"),
    ({"model_type": "llama"}, "model_type"),
    ({"architectures": ["LlamaForCausalLM"]}, "architectures"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"attn_logit_softcapping": 30.0}, "attn_logit_softcapping"),
    ({"final_logit_softcapping": 30.0}, "final_logit_softcapping"),
    ({"num_local_experts": 8}, "num_local_experts"),
    ({"n_routed_experts": 8}, "n_routed_experts"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"num_experts_per_tok": 9}, "experts"),
    ({"decoder_sparse_step": 0}, "experts"),
    ({"mlp_only_layers": [5]}, "experts"),
    ({"shared_expert_intermediate_size": 0}, "experts"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_refusals_name_the_feature(patch, feature):
    with pytest.raises(Unsupported) as e:
        config_from_dict({**TINY_A, **patch})
    assert e.value.feature == feature


@pytest.mark.parametrize("patch", [
    {"num_attention_heads": 0}, {"num_key_value_heads": 3}, {"head_dim": 15}, {"hidden_size": 0},
    {"vocab_size": 0}, {"rms_norm_eps": 0.0}, {"rope_theta": -1.0}, {"sliding_window": 0},
    {"max_position_embeddings": 0}, {"num_hidden_layers": 0}, {"hidden_size": "64"},
    {"head_dim": None, "hidden_size": 66},
])
def test_invalid_values(patch):
    with pytest.raises(InvalidConfig):
        config_from_dict({**TINY_A, **patch})


def test_missing_required_key_and_disagreement():
    with pytest.raises(InvalidConfig, match="moe_intermediate_size"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "moe_intermediate_size"})
    with pytest.raises(InvalidConfig):
        config_from_dict({k: v for k, v in TINY_A.items() if k not in ("architectures", "model_type")})


def test_hidden_act_swish_is_silu_and_round_trip(tmp_path):
    c = config_from_dict({**TINY_B, "hidden_act": "swish"})
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    again = config_from_json(tmp_path)
    assert again == c
    assert config_from_json((tmp_path / "config.json").read_bytes()) == c


def test_the_plan_carries_the_checkpoint_names_and_the_parts_spell_none():
    """Tensor names are data of the plan: another name table gives other parameter names from the same parts."""
    import dataclasses
    import torch
    from esp_b200.config import config_from_dict
    from esp_b200.config.plan import AttentionNames, MoeNames, SwiGluNames
    from esp_b200.engine.model import DecoderModel
    from esp_b200.parts import Runtime
    from esp_b200.weights import InitSpec
    import sys, pathlib
    sys.path.insert(0, str(pathlib.Path(__file__).parent))
    from tiny import TINY_A
    plan = config_from_dict(TINY_A).plan()
    names = {s.name for part in DecoderModel(plan, Runtime(None, torch.float32)).all_parts() for s in part.param_specs()}
    assert "model.layers.0.self_attn.q_proj.weight" in names and "model.layers.1.mlp.experts.3.down_proj.weight" in names
    other_mlp = SwiGluNames("w1.weight", "w3.weight", "w2.weight")
    plan.blocks = [dataclasses.replace(
        b, mixer=dataclasses.replace(b.mixer, names=AttentionNames("wq", "wk", "wv", "wo", ".w", ".b")),
        ffn=dataclasses.replace(b.ffn, names=MoeNames("router.weight", "shared_gate.weight", "shared.", "expert_{e}.", other_mlp)))
        for b in plan.blocks]
    renamed = {s.name for part in DecoderModel(plan, Runtime(None, torch.float32)).all_parts() for s in part.param_specs()}
    assert {"model.layers.0.self_attn.wq.w", "model.layers.0.self_attn.wk.b", "model.layers.1.mlp.expert_3.w2.weight",
            "model.layers.0.mlp.router.weight", "model.layers.1.mlp.shared.w1.weight"} <= renamed
    assert len(renamed) == len(names)
    # a role of its own gets its rule from the spec; an unknown one is refused by name
    assert InitSpec(roles=(("decay", 0.5, 0.1),)).mean_std("decay") == (0.5, 0.1)
    from esp_b200.errors import InvalidConfig
    import pytest
    with pytest.raises(InvalidConfig, match="decay"):
        InitSpec().mean_std("decay")


def test_which_grouped_kernel_a_step_takes():
    """The weight-streaming kernel while no expert can have more than eight rows and the step has fewer than
    128 (token, expert) rows; the TMA + tcgen05 kernel beyond either bound, and never for 32-bit operands."""
    import torch
    from esp_b200.parts import linear
    a = torch.empty(4, 64, dtype=torch.bfloat16)
    w = torch.empty(3, 32, 64, dtype=torch.bfloat16)
    assert not linear.grouped_uses_tc05(a, w, 32, 8)
    assert linear.grouped_uses_tc05(a, w, 36, 9)
    assert linear.grouped_uses_tc05(a, w, 128, 8)
    assert not linear.grouped_uses_tc05(a, w, 127)
    assert not linear.grouped_uses_tc05(a.float(), w.float(), 4096, 1024)
    assert not linear.grouped_uses_tc05(a[:, :60], w[:, :, :60], 4096, 1024)      # K no multiple of 8


def test_how_many_positions_a_block_of_the_decode_attention_takes():
    """Whole pages, never fewer than the minimum, few enough splits that one round of blocks holds them when the
    rows are few, and the choices that were measured (16 key/value heads of 128, 4,096 positions)."""
    from esp_b200.csrc import ops
    room = 148 * ops.ATTN_DECODE_BLOCKS_PER_SM[128]
    for rows, kv, positions in [(1, 16, 4096), (2, 16, 4096), (5, 16, 4096), (8, 16, 4096), (16, 16, 4096), (1, 4, 32000),
                                (8, 4, 32000), (3, 7, 1000), (1, 1, 64), (1, 1, 65), (64, 16, 256), (7, 3, 12345)]:
        split = ops.attn_decode_split(rows, kv, positions)
        assert split % 64 == 0 and split >= min(128 if positions <= 4096 else 256, 64 * ((positions + 63) // 64))
        if rows * kv * 2 <= room:
            assert rows * kv * ((positions + split - 1) // split) <= room, (rows, kv, positions, split)
    assert [ops.attn_decode_split(b, 16, 4096) for b in (1, 2, 4, 8, 16, 32, 48, 64)] == [128, 256, 512, 1024, 2048, 4096, 1408, 4096]
    assert ops.attn_decode_split(1, 4, 32000) == 256 and ops.attn_decode_split(1, 16, 8000) == 256
