"""Plain, slow Qwen2-MoE decoder used as the oracle of the test suite.

Whole sequences, no cache, one function per part, numpy only.  Nothing here is
shared with the product path under ``esp_b200/``: it has its own safetensors
reader, its own configuration reading and its own sampler.

The reference project (merely-made/esp) is Rust on the Burn tensor library and
cannot be compiled or imported in a Python process, so this file rests on the
reference's formulas, cited per function as ``file:line`` within that project.
It is anchored on the two Qwen2-MoE checkpoints that the reference ships with
independently recorded outputs (``tests/golden/``, see ``test_plain.py``).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------
# reading a model folder
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "F64": np.float64}


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path) -> dict[str, np.ndarray]:
    """8-byte little-endian header length, JSON header, raw little-endian data
    (crates/esp/src/infer/decoder/checkpoint.rs:47-158).  Everything is widened
    to float32 as the reference does at load
    (crates/esp/src/infer/decoder/weight_format.rs:110-133)."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[base + lo : base + hi]
        if meta["dtype"] == "BF16":
            arr = _bf16_to_f32(np.frombuffer(raw, dtype=np.uint16))
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[meta["dtype"]]).astype(np.float32)
        out[name] = arr.reshape(meta["shape"])
    return out


def read_config(path) -> dict:
    return read_config_dict(json.loads(Path(path).read_text()))


def read_config_dict(c: dict) -> dict:
    """config.json's keys with the reference's defaults filled in
    (crates/esp/src/infer/decoder/config.rs:36-51, :322-386, :434-446)."""
    c = dict(c)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", False)
    c.setdefault("norm_topk_prob", False)
    c.setdefault("decoder_sparse_step", 1)
    c.setdefault("mlp_only_layers", [])
    c.setdefault("use_sliding_window", None)
    c.setdefault("sliding_window", None)
    c.setdefault("max_window_layers", 28)
    c.setdefault("layer_types", None)
    return c


def load_model(folder) -> tuple[dict, dict[str, np.ndarray]]:
    folder = Path(folder)
    return read_config(folder / "config.json"), read_safetensors(folder / "model.safetensors")


def layer_is_moe(c: dict, i: int) -> bool:
    """crates/esp/src/infer/decoder/config.rs:460-464.  A configuration without experts (the reference's
    dense ``qwen2`` checkpoint, which shares the attention code and is used here to pin the window) has
    dense layers only."""
    if not c.get("num_experts"):
        return False
    return i not in c["mlp_only_layers"] and (i + 1) % c["decoder_sparse_step"] == 0


def layer_window(c: dict, i: int):
    """crates/esp/src/infer/decoder/config.rs:466-485: ``layer_types``, when present, decides layer by
    layer; else ``use_sliding_window`` and ``max_window_layers`` (the qwen2 / qwen2_moe branch)."""
    if c.get("layer_types") is not None:
        return c["sliding_window"] if c["layer_types"][i] == "sliding_attention" else None
    if c["use_sliding_window"] is False:
        return None
    if c.get("model_type") not in ("qwen2", "qwen3", "qwen2_moe"):
        # every other family the reference reads: a window, when given, holds for every layer (used here only
        # for its dense ``mistral`` checkpoint, whose head size differs from width / heads)
        return c["sliding_window"]
    if c["use_sliding_window"] is True and i >= c["max_window_layers"]:
        return c["sliding_window"]
    return None


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def rms_norm(x, gamma, eps):
    """y = x * rsqrt(mean(x^2) + eps) * gamma
    (crates/esp/src/infer/decoder/layer.rs:27-33, :125, :150)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + x.dtype.type(eps)) * gamma


def rope_angles(positions, head_dim, theta):
    """Split-half rotary angles, frequencies and angles in float32
    (crates/esp/src/infer/decoder/attention.rs:58-95): f_i = 1/theta^(2i/hd),
    angle = float32(p) * f_i."""
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * i) / np.float32(head_dim))).astype(np.float32)
    ang = np.asarray(positions, dtype=np.float32)[:, None] * freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def apply_rope(x, cos, sin):
    """x: [T, heads, hd]; o_i = x_i cos - x_{i+h} sin; o_{i+h} = x_{i+h} cos + x_i sin
    (crates/esp/src/infer/decoder/attention.rs:99-123)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c = cos[:, None, :].astype(x.dtype)
    s = sin[:, None, :].astype(x.dtype)
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def attention(c, w, prefix, x, window):
    """GQA attention of one layer over a whole sequence x [T, H]
    (crates/esp/src/infer/decoder/attention.rs:292-404): q/k/v with bias (where the checkpoint has one),
    rotary on q and k, scores divided by sqrt(hd) after the product, key j of
    query a masked iff j > a or (window and a - j >= window), softmax, PV,
    o_proj without bias."""
    T = x.shape[0]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    def project(name):      # the bias is added where the checkpoint has one (the Qwen2 families do, always)
        y = x @ w[prefix + name + ".weight"].T
        return y + w[prefix + name + ".bias"] if prefix + name + ".bias" in w else y

    q, k, v = project("q_proj"), project("k_proj"), project("v_proj")
    q = q.reshape(T, nh, hd)
    k = k.reshape(T, nkv, hd)
    v = v.reshape(T, nkv, hd)
    cos, sin = rope_angles(np.arange(T), hd, c["rope_theta"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    group = nh // nkv
    a = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    masked = j > a
    if window is not None:
        masked |= (a - j) >= window
    out = np.empty((T, nh, hd), dtype=x.dtype)
    for h in range(nh):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        s = (q[:, h, :] @ kh.T) / x.dtype.type(np.sqrt(np.float32(hd)))
        s = np.where(masked, -np.inf, s)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ vh
    return out.reshape(T, nh * hd) @ w[prefix + "o_proj.weight"].T


def swiglu(x, wg, wu, wd):
    """down(silu(gate x) * (up x)) (crates/esp/src/infer/decoder/moe.rs:87-89)."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1.0 + np.exp(-g))) * u) @ wd.T


def dense_mlp(w, prefix, x):
    """crates/esp/src/infer/decoder/moe.rs:143-148"""
    return swiglu(x, w[prefix + "gate_proj.weight"], w[prefix + "up_proj.weight"], w[prefix + "down_proj.weight"])


def route(c, w, prefix, x):
    """Router: float32 softmax over all experts, top-k by probability with ties
    to the lower id, optional renormalisation
    (crates/esp/src/infer/decoder/moe.rs:156-181).  Returns ids [T,k] and
    weights [T,k] and the full probabilities."""
    logits = (x @ w[prefix + "gate.weight"].T).astype(np.float32)
    logits = logits - logits.max(axis=-1, keepdims=True)
    p = np.exp(logits)
    p = p / p.sum(axis=-1, keepdims=True)
    k = c["num_experts_per_tok"]
    ids = np.argsort(-p, axis=-1, kind="stable")[:, :k]
    return ids, p


def moe_block(c, w, prefix, x, forced_ids=None, record=None):
    """Sparse block: routed experts summed in ascending expert id, each output
    scaled by its routing weight, plus the shared expert scaled by
    sigmoid(x . w_shared_gate) (crates/esp/src/infer/decoder/moe.rs:182-255).
    ``forced_ids`` [T,k] replaces the top-k choice (weights still come from this
    function's own probabilities); ``record`` receives (ids, probabilities)."""
    ids, p = route(c, w, prefix, x)
    if record is not None:
        record.append((ids.copy(), p.copy()))
    if forced_ids is not None:
        ids = np.asarray(forced_ids)
    out = np.zeros_like(x)
    chosen = np.zeros(p.shape, dtype=bool)
    np.put_along_axis(chosen, ids, True, axis=-1)
    if c["norm_topk_prob"]:
        s = np.where(chosen, p, np.float32(0.0)).sum(axis=-1, dtype=np.float32)
    else:
        s = np.ones(p.shape[0], dtype=np.float32)
    for e in range(p.shape[1]):  # ascending expert id
        rows = np.nonzero(chosen[:, e])[0]
        if rows.size == 0:
            continue
        ep = f"{prefix}experts.{e}."
        y = swiglu(x[rows], w[ep + "gate_proj.weight"], w[ep + "up_proj.weight"], w[ep + "down_proj.weight"])
        out[rows] += y * (p[rows, e] / s[rows]).astype(x.dtype)[:, None]
    sp = prefix + "shared_expert."
    shared = swiglu(x, w[sp + "gate_proj.weight"], w[sp + "up_proj.weight"], w[sp + "down_proj.weight"])
    gate = 1.0 / (1.0 + np.exp(-(x @ w[prefix + "shared_expert_gate.weight"].T)))
    return out + gate * shared


def decoder_layer(c, w, i, x, forced_ids=None, record=None):
    """Pre-norm block with two residuals
    (crates/esp/src/infer/decoder/layer.rs:115-153)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
    x = x + attention(c, w, p + "self_attn.", h, layer_window(c, i))
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
    if layer_is_moe(c, i):
        return x + moe_block(c, w, p + "mlp.", h, forced_ids, record)
    return x + dense_mlp(w, p + "mlp.", h)


def forward_logits(c, w, ids, dtype=np.float32, forced_routing=None, routing_record=None):
    """Logits [T, V] of a whole sequence, every position
    (crates/esp/src/infer/decoder/model.rs:468-473, :541-666).  ``forced_routing``
    maps layer index -> ids [T,k]; ``routing_record`` (a dict) receives, per MoE
    layer, (ids, probabilities)."""
    w = {k: v.astype(dtype, copy=False) for k, v in w.items()}
    x = w["model.embed_tokens.weight"][np.asarray(ids)]
    for i in range(c["num_hidden_layers"]):
        rec = None
        if routing_record is not None and layer_is_moe(c, i):
            rec = []
        forced = forced_routing.get(i) if forced_routing else None
        x = decoder_layer(c, w, i, x, forced, rec)
        if rec:
            routing_record[i] = rec[0]
    x = rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]
    return (x @ head.T).astype(np.float32)


# --------------------------------------------------------------------------
# choosing tokens
# --------------------------------------------------------------------------

def argmax_lower_id(row) -> int:
    """Greedy choice, lower id on ties
    (crates/esp/src/infer/decoder/generate.rs:70-79, provider.rs:809-815)."""
    return int(np.argmax(row))


class SplitMix64:
    """crates/esp/src/infer/decoder/sample.rs:23-52"""
    M = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = seed & self.M

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.M
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.M
        return z ^ (z >> 31)

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)

    def skip(self, draws: int):
        self.state = (self.state + 0x9E3779B97F4A7C15 * draws) & self.M


def sample_row(row, temperature, top_p, rng: SplitMix64) -> int:
    """Temperature weights in float32, walk in descending weight (ties: lower
    id first), optional nucleus cut, inverse-CDF draw with one draw per token
    (crates/esp/src/infer/decoder/sample.rs:83-121)."""
    row = np.asarray(row, dtype=np.float32)
    inv_t = np.float32(1.0) / np.float32(temperature)
    wts = np.exp((row - row.max()) * inv_t).astype(np.float32)
    order = np.argsort(-wts, kind="stable")
    sw = wts[order]
    if top_p is not None:
        total = np.float32(0.0)
        for x in sw:
            total = np.float32(total + x)
        target = np.float32(total * np.float32(min(max(top_p, 0.0), 1.0)))
        mass = np.float32(0.0)
        keep = 0
        for i, x in enumerate(sw):
            mass = np.float32(mass + x)
            keep = i + 1
            if mass >= target:
                break
        keep = max(keep, 1)
        sw, order = sw[:keep], order[:keep]
    total = np.float32(0.0)
    for x in sw:
        total = np.float32(total + x)
    u = np.float32(np.float32(rng.next_f64()) * total)
    for idx, x in zip(order, sw):
        u = np.float32(u - x)
        if u <= 0.0:
            return int(idx)
    return int(order[-1])


def generate(c, w, prompt, max_new, eos=(), temperature=0.0, top_p=None, seed=0, dtype=np.float32):
    """Full recomputation per token; a stop token ends the sequence, is not
    emitted and costs one draw (crates/esp/src/infer/decoder/generate.rs:134-170,
    :267-289)."""
    ids = list(prompt)
    out = []
    rng = SplitMix64(seed)
    for _ in range(max_new):
        row = forward_logits(c, w, ids, dtype)[-1]
        tok = argmax_lower_id(row) if temperature == 0.0 else sample_row(row, temperature, top_p, rng)
        if tok in eos:
            break
        out.append(tok)
        ids.append(tok)
    return out
