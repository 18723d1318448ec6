"""The two tiny configurations of the test suite.  They differ in every size
and option: head counts and grouping, head size, widths that are no power of
two, number of layers, vocabulary, eps, rope base, window, experts, top-k,
renormalisation, dense layers, tying, initialisation."""
import json
import os
from pathlib import Path

import numpy as np

TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 128,
    "intermediate_size": 96, "num_experts": 4, "num_experts_per_tok": 2, "norm_topk_prob": False,
    "moe_intermediate_size": 32, "shared_expert_intermediate_size": 64, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": None, "tie_word_embeddings": False,
}
INIT_A = dict(weight_std=0.02, bias_std=0.02, norm_std=0.01)
PROMPTS_A = (5, 11, 17)

TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 24,
    "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 256,
    "intermediate_size": 128, "num_experts": 6, "num_experts_per_tok": 3, "norm_topk_prob": True,
    "moe_intermediate_size": 48, "shared_expert_intermediate_size": 80, "decoder_sparse_step": 2,
    "mlp_only_layers": [0], "use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1,
    "tie_word_embeddings": True,
}
INIT_B = dict(weight_std=0.05, bias_std=0.0, norm_std=0.0)
PROMPTS_B = (1, 7, 23, 40)

# Sizes that fit none of the fast kernels' alignments: a width that is no multiple of 8, five heads whose
# size times count differs from the width, an odd vocabulary, intermediate sizes that are multiples of 4 only.
TINY_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 24,
    "vocab_size": 301, "rope_theta": 50000.0, "rms_norm_eps": 2e-6, "max_position_embeddings": 160,
    "intermediate_size": 44, "num_experts": 5, "num_experts_per_tok": 2, "norm_topk_prob": True,
    "moe_intermediate_size": 20, "shared_expert_intermediate_size": 36, "decoder_sparse_step": 1,
    "mlp_only_layers": [1], "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 0,
    "tie_word_embeddings": False,
}
INIT_C = dict(weight_std=0.04, bias_std=0.03, norm_std=0.02)

CASES = {"A": (TINY_A, INIT_A), "B": (TINY_B, INIT_B), "C": (TINY_C, INIT_C)}


def make_folder(tmp: Path, case: str, seed: int = 1234, store: str = "bfloat16", **overrides) -> Path:
    """Writes config.json and model.safetensors of a tiny case into ``tmp``."""
    from esp_b200.config import config_from_dict
    from esp_b200.weights import InitSpec, write_model_folder
    raw, init = CASES[case]
    raw = {**raw, **overrides}
    folder = Path(tmp) / f"tiny_{case}_{store}"
    write_model_folder(config_from_dict(raw), seed, folder, store, InitSpec(**init))
    return folder


def random_config(rng: np.random.Generator) -> dict:
    """A configuration drawn from the sizes the architecture allows: head sizes in steps of 16 from 16 to 128, one
    to three key/value heads with one to five query heads each, widths that are and are not multiples of 8, odd
    vocabularies, one to three layers, dense layers among them, windows from 5 to 130 positions, tying."""
    hd = int(rng.choice([16, 32, 48, 64, 80, 128]))
    nkv = int(rng.choice([1, 2, 3]))
    nh = nkv * int(rng.choice([1, 2, 4, 5]))
    layers = int(rng.choice([1, 2, 3]))
    experts = int(rng.choice([3, 4, 7, 8, 12]))
    window = bool(rng.integers(0, 2))
    return {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
        "num_hidden_layers": layers, "hidden_size": int(rng.choice([64, 72, 100, 128, 136, 200])),
        "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
        "vocab_size": int(rng.choice([97, 256, 301, 512])), "rope_theta": float(rng.choice([1e4, 1e6, 5e4])),
        "rms_norm_eps": float(rng.choice([1e-6, 1e-5])), "max_position_embeddings": 1024,
        "intermediate_size": int(rng.choice([40, 64, 96, 136])), "num_experts": experts,
        "num_experts_per_tok": int(rng.integers(1, min(experts, 5) + 1)), "norm_topk_prob": bool(rng.integers(0, 2)),
        "moe_intermediate_size": int(rng.choice([16, 24, 40, 64])),
        "shared_expert_intermediate_size": int(rng.choice([24, 32, 56, 128])),
        "decoder_sparse_step": int(rng.choice([1, 1, 2])),
        "mlp_only_layers": [0] if (layers > 1 and rng.integers(0, 3) == 0) else [],
        "use_sliding_window": window, "sliding_window": int(rng.choice([5, 17, 64, 70, 130])) if window else None,
        "max_window_layers": int(rng.integers(0, layers)) if window else 28,
        "tie_word_embeddings": bool(rng.integers(0, 2)),
    }


def random_ids(rng: np.random.Generator, n: int, vocab: int) -> list:
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def repo_root() -> Path:
    return Path(__file__).resolve().parent.parent
