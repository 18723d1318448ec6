"""Decode and prefill throughput of the Qwen1.5-MoE-A2.7B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--context C] [--layers L]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch B
(default 8) with the timed steps ending at context C (default 4096), timed on
the device with CUDA events; ``e2e`` is the same through the Python entry
point (host token ids in, host tokens out, every step).  ``prefill`` is one
2,048-token prompt; ``roofline`` compares the bytes a decode step has to read
(every weight it uses once, and the cache of the live requests) with the
measured HBM bandwidth; ``points`` holds decode at batch 1 and 64.  Weights are
random (N(0, 0.02)), token ids synthetic and uniform.  A decode step reads far
more than the 126 MB of L2 (over 10 GB of weights and cache), so consecutive
timed steps cannot reuse each other's data from L2.

``--impl reference``: the reference (merely-made/esp) is a Rust crate whose GPU
path is a graphics API; it cannot be installed or run here, so that arm
prints its ``unavailable`` line.
"""
import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "hidden_act": "silu",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "intermediate_size": 5632, "num_experts": 60, "num_experts_per_tok": 4,
    "norm_topk_prob": False, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": None,
    "tie_word_embeddings": False,
}
FULL_LAYERS = 24
# the second shape that the reference's real-model gates use: Qwen2-57B-A14B layer sizes (--shape 57b-a14b)
Q57B = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
            max_position_embeddings=32768, intermediate_size=18944, num_experts=64, num_experts_per_tok=8,
            moe_intermediate_size=2560, shared_expert_intermediate_size=20480)
SHAPES = {"a2.7b": (A27B, "Qwen1.5-MoE-A2.7B layer sizes"), "57b-a14b": (Q57B, "Qwen2-57B-A14B layer sizes")}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(r[0]))
                mx.append(int(r[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, r[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, layers):
    """Per-token FLOPs without attention scores, and weight bytes of the parts of a layer (bfloat16)."""
    H, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, Im, Is, V = (cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"],
                       cfg["shared_expert_intermediate_size"], cfg["vocab_size"])
    attn_w = H * (nh + 2 * nkv) * hd + nh * hd * H
    layer_fixed = attn_w + E * H + H + 3 * H * Is          # attention, router, shared gate, shared expert
    expert_w = 3 * H * Im
    flops_token = layers * 2 * (attn_w + E * H + H + 3 * H * Is + k * expert_w)
    return {"layer_fixed_bytes": 2 * layer_fixed, "expert_bytes": 2 * expert_w, "head_bytes": 2 * V * H,
            "flops_token": flops_token, "attn_flops_per_key": layers * 4 * nh * hd,
            "kv_bytes_token": layers * 2 * nkv * hd * 2, "head_flops_row": 2 * V * H}


def timed_steps(torch, fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps


def decode_run(torch, engine, batch, context, warmup, steps, vocab, seed):
    """Prefills ``batch`` prompts so that warmup + steps decode steps end at
    ``context``, then times the decode steps on the device.  Returns
    (ms per step, distinct experts per layer, slots)."""
    import numpy as np
    from esp_b200.engine import StepEntry
    rng = np.random.default_rng(seed)
    prompt_len = context - warmup - steps - 1
    slots = [engine.open() for _ in range(batch)]
    for s in slots:                      # one prompt per step keeps the prefill's scratch small
        toks = rng.integers(0, vocab, prompt_len).tolist()
        engine.step([StepEntry(s, toks, [])])
    torch.cuda.synchronize()
    temps, tops = [0.0] * batch, [None] * batch

    def one():
        toks = rng.integers(0, vocab, batch).tolist()
        engine.step_and_pick([StepEntry(s, [t], [0]) for s, t in zip(slots, toks)], temps, tops)

    engine.rt.record_routing = True
    aux = {}
    engine.step([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, rng.integers(0, vocab, batch))], aux)
    engine.rt.record_routing = False
    distinct = [int(torch.unique(ids).numel()) for _p, _r, ids, _w, _pr in aux.get("routing", [])]
    ms = timed_steps(torch, one, warmup, steps)
    return ms, (sum(distinct) / len(distinct) if distinct else 0.0), slots, prompt_len


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="esp_b200")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--shape", default="a2.7b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill measurement (for profiling decode)")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "merely-made/esp is a Rust crate (no cargo/rustc here, pip "
                          "finds neither setup.py nor pyproject.toml) and its only GPU path is a graphics API (wgpu): "
                          "unavailable on this box"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures a one-GPU library: --gpus {a.gpus} is not supported (run with --gpus 1)")
        return 2
    a.warmup = max(a.warmup, 3)

    import numpy as np
    import torch
    from esp_b200.config import config_from_dict
    from esp_b200.csrc import ops
    from esp_b200.engine import Engine, StepEntry
    from esp_b200.provider import DecoderProvider, GenerationRequest
    from esp_b200.weights import InitSpec

    pk = peaks()
    shape, shape_name = SHAPES[a.shape]
    full_layers = shape["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    raw = dict(shape, num_hidden_layers=a.layers)
    cfg = config_from_dict(raw)
    nums = model_numbers(raw, a.layers)
    vocab = raw["vocab_size"]
    biggest = max(a.batch, 1 if a.no_points else 64)
    engine = Engine.from_random(cfg, seed=0, init=InitSpec(0.02, 0.02, 0.0), dtype="bfloat16",
                                max_tokens=biggest * (a.context + 64), max_slots=biggest + 2)
    torch.cuda.synchronize()

    # ---- prefill of one 2,048-token prompt --------------------------------------
    rng = np.random.default_rng(1)
    T = 2048

    def prefill_once():
        s = engine.open()
        engine.step([StepEntry(s, rng.integers(0, vocab, T).tolist(), [T - 1])])
        engine.close(s)

    prefill = None
    if not a.no_prefill:
        ms_prefill = timed_steps(torch, prefill_once, 3, 5)
        prefill_flops = nums["flops_token"] * T + nums["attn_flops_per_key"] * T * (T + 1) / 2 + nums["head_flops_row"]
        prefill = {"value": round(T / ms_prefill * 1e3, 1), "tokens": T, "ms": round(ms_prefill, 3),
                   "frac": round(prefill_flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at the headline batch ---------------------------------------------
    launches_before = ops.launch_count()
    with ClockSampler() as clocks:
        ms_step, distinct, slots, prompt_len = decode_run(torch, engine, a.batch, a.context, a.warmup, a.steps, vocab, 2)
    launches = ops.launch_count() - launches_before
    for s in slots:
        engine.close(s)
    ctx_mean = a.context - (a.steps + 1) / 2
    step_bytes = (a.layers * (nums["layer_fixed_bytes"] + distinct * nums["expert_bytes"]) + nums["head_bytes"]
                  + a.batch * ctx_mean * nums["kv_bytes_token"])
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    value = a.batch / ms_step * 1e3

    # ---- the same through the Python entry point ------------------------------------
    e2e = None
    if not a.no_e2e:
        prov = DecoderProvider(engine, None, max_batch=a.batch)
        n_new = a.warmup + a.steps + 1
        reqs = [GenerationRequest(prompt_ids=rng.integers(0, vocab, a.context - n_new).tolist(), max_tokens=n_new)
                for _ in range(a.batch)]
        marks = {}

        def on_token(i, tok):
            if i == a.batch - 1:          # the last sequence of a step: the step's tokens are on the host
                marks[len(marks)] = time.perf_counter()
            return False

        prov.generate(reqs, on_token)
        t0, t1 = marks[a.warmup], marks[a.warmup + a.steps]
        h2d = engine.staged_bytes         # the last step's staged arrays: ids, positions, page tables, sampling options
        e2e = {"value": round(a.batch * a.steps / (t1 - t0), 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4 * (a.batch + 1)}

    # ---- decode at batch 1 and 64 --------------------------------------------------------
    points = {}
    if not a.no_points:
        for b in (1, 64):
            ms_b, _d, sl, _p = decode_run(torch, engine, b, a.context, a.warmup, max(8, a.steps // 2), vocab, 3 + b)
            for s in sl:
                engine.close(s)
            points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)

    line = {
        "metric": f"decode tok/s at batch {a.batch}", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
        "impl": "esp_b200",
        "config": {"model": shape_name, "layers": a.layers, "layers_of_model": full_layers,
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "vocab": vocab,
                   "experts": raw["num_experts"], "top_k": raw["num_experts_per_tok"],
                   "moe_intermediate": raw["moe_intermediate_size"],
                   "shared_intermediate": raw["shared_expert_intermediate_size"], "global_batch": a.batch,
                   "seq_len": a.context, "prompt_len": prompt_len, "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (a step reads >10 GB)", "distinct_experts_per_layer": round(distinct, 1)},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(), "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
