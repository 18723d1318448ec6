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
            "kv_bytes_token": layers * 2 * nkv * hd * 2, "head_flops_row": 2 * V * H,
            "dense_flops_token_layer": 2 * (attn_w + E * H + H + 3 * H * Is), "expert_flops_token_layer": 2 * k * expert_w,
            "n_experts": E}


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
    (ms per step, distinct experts per sparse layer averaged over the timed steps, slots, prompt length)."""
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

    for _ in range(warmup):              # the steps that size scratch, load kernels and capture the graph
        one()
    before = engine.counters()
    ms = timed_steps(torch, one, 0, steps)
    after = engine.counters()
    sparse_layers = sum(1 for b in engine.plan.blocks if getattr(b.ffn, "kind", "") == "moe_swiglu_shared")
    reads = after.get("expert_reads", 0) - before.get("expert_reads", 0)
    distinct = reads / (steps * sparse_layers) if sparse_layers else 0.0
    return ms, distinct, slots, prompt_len


def decode_roofline(nums, layers, batch, context, steps, distinct, ms, pk):
    """Bytes a decode step has to read (every weight it uses once, and the cache of the live requests)
    against the HBM peak."""
    ctx_mean = context - (steps + 1) / 2
    step_bytes = (layers * (nums["layer_fixed_bytes"] + distinct * nums["expert_bytes"]) + nums["head_bytes"]
                  + batch * ctx_mean * nums["kv_bytes_token"])
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}


def prefill_numbers(nums, layers, T, ms, pk):
    """``frac``: all FLOPs of the step over the tensor-core peak.  ``frac_of_bound``: against the sum over the
    step's products of max(FLOPs / peak, weight bytes / HBM peak): at one prompt of 2,048 tokens the routed
    experts are bound by streaming their weights, not by arithmetic."""
    flops = nums["flops_token"] * T + nums["attn_flops_per_key"] * T * (T + 1) / 2 + nums["head_flops_row"]
    peak_f, peak_b = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    dense = max(nums["dense_flops_token_layer"] * T / peak_f, nums["layer_fixed_bytes"] / peak_b)
    routed = max(nums["expert_flops_token_layer"] * T / peak_f, nums["n_experts"] * nums["expert_bytes"] / peak_b)
    attn = nums["attn_flops_per_key"] * T * (T + 1) / 2 / peak_f
    head = max(nums["head_flops_row"] / peak_f, nums["head_bytes"] / peak_b)
    bound_ms = (layers * (dense + routed) + attn + head) * 1e3
    return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
            "frac": round(flops / (ms * 1e-3) / peak_f, 4), "bound_ms": round(bound_ms, 3),
            "frac_of_bound": round(bound_ms / ms, 4)}


def measure_shape(torch, raw, layers, batch, context, steps, warmup, pk, points=(1, 64), e2e=True, prefill=True,
                  clocks=None, prefill_tokens=2048):
    """Builds the model with random weights and measures prefill, decode at ``batch``, the same through the
    entry point, and decode at ``points``.  Returns a dict of results; the engine is freed before returning."""
    import gc
    import numpy as np
    from esp_b200.config import config_from_dict
    from esp_b200.csrc import ops
    from esp_b200.engine import Engine, StepEntry
    from esp_b200.provider import DecoderProvider, GenerationRequest
    from esp_b200.weights import InitSpec

    cfg = config_from_dict(dict(raw, num_hidden_layers=layers))
    nums = model_numbers(raw, layers)
    vocab = raw["vocab_size"]
    biggest = max([batch, *points])
    engine = Engine.from_random(cfg, seed=0, init=InitSpec(0.02, 0.02, 0.0), dtype="bfloat16",
                                max_tokens=max(biggest * (context + 64), prefill_tokens + 64), max_slots=biggest + 2)
    torch.cuda.synchronize()
    out = {}
    rng = np.random.default_rng(1)
    T = prefill_tokens

    def prefill_once():
        s = engine.open()
        engine.step([StepEntry(s, rng.integers(0, vocab, T).tolist(), [T - 1])])
        engine.close(s)

    if prefill:
        out["prefill"] = prefill_numbers(nums, layers, T, timed_steps(torch, prefill_once, 3, 5), pk)

    launches_before = ops.launch_count()
    if clocks is not None:
        with clocks:
            ms_step, distinct, slots, prompt_len = decode_run(torch, engine, batch, context, warmup, steps, vocab, 2)
    else:
        ms_step, distinct, slots, prompt_len = decode_run(torch, engine, batch, context, warmup, steps, vocab, 2)
    out["gpu_launches"] = ops.launch_count() - launches_before
    for s in slots:
        engine.close(s)
    out.update(ms_per_step=ms_step, value=batch / ms_step * 1e3, distinct=distinct, prompt_len=prompt_len,
               roofline=decode_roofline(nums, layers, batch, context, steps, distinct, ms_step, pk))

    if e2e:
        prov = DecoderProvider(engine, None, max_batch=batch)
        n_new = warmup + steps + 1
        reqs = [GenerationRequest(prompt_ids=rng.integers(0, vocab, context - n_new).tolist(), max_tokens=n_new)
                for _ in range(batch)]
        marks = {}

        def on_token(i, tok):
            if i == batch - 1:            # the last sequence of a step: the step's tokens are on the host
                marks[len(marks)] = time.perf_counter()
            return False

        prov.generate(reqs, on_token)
        t0, t1 = marks[warmup], marks[warmup + steps]
        h2d = engine.staged_bytes         # the last step's staged arrays: ids, positions, page tables, sampling options
        out["e2e"] = {"value": round(batch * steps / (t1 - t0), 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": 4 * (batch + 1)}

    out["points"], out["points_detail"] = {}, {}
    for b in points:
        n = max(8, steps // 2)
        ms_b, d_b, sl, _p = decode_run(torch, engine, b, context, warmup, n, vocab, 3 + b)
        for s in sl:
            engine.close(s)
        out["points"][f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
        out["points_detail"][f"decode_b{b}"] = {
            "ms": round(ms_b, 4), "distinct_experts_per_layer": round(d_b, 1),
            "hbm_frac": decode_roofline(nums, layers, b, context, n, d_b, ms_b, pk)["frac"]}
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


def fp32_cuttings(torch, raw, layers, n_prompts=16, longest=1024, decoded=64, seed=7):
    """The true 32-bit path at the headline layer sizes: ``n_prompts`` requests with prompt lengths uniform in
    [1, longest] and ``decoded`` further given tokens each, run three ways: every request alone and whole; its
    prompt, then its tokens one by one; all prompts as one batch, then one token of each per step.  The logits
    at the last ``decoded`` + 1 positions of every request are compared on the device, bit for bit."""
    import gc
    import numpy as np
    from esp_b200.config import config_from_dict
    from esp_b200.engine import Engine, StepEntry
    from esp_b200.weights import InitSpec

    t_start = time.perf_counter()
    cfg = config_from_dict(dict(raw, num_hidden_layers=layers))
    rng = np.random.default_rng(seed)
    vocab = raw["vocab_size"]
    plens = [int(n) for n in rng.integers(1, longest + 1, n_prompts)]
    reqs = [rng.integers(0, vocab, n + decoded).tolist() for n in plens]
    tokens = sum((len(r) + 63) // 64 * 64 for r in reqs)
    engine = Engine.from_random(cfg, seed=0, init=InitSpec(0.02, 0.02, 0.0), dtype="float32", stored_dtype="bfloat16",
                                max_tokens=tokens + 64, max_slots=n_prompts + 1)
    torch.cuda.synchronize()
    t_built = time.perf_counter()

    def whole():
        rows = []
        for r, n in zip(reqs, plens):
            s = engine.open()
            rows.append(engine.step([StepEntry(s, r, list(range(n - 1, len(r))))]))
            engine.close(s)
        return rows

    def one_by_one():
        rows = []
        for r, n in zip(reqs, plens):
            s = engine.open()
            got = [engine.step([StepEntry(s, r[:n], [n - 1])])]
            got += [engine.step([StepEntry(s, [t], [0])]) for t in r[n:]]
            engine.close(s)
            rows.append(torch.cat(got))
        return rows

    def batched():
        slots = [engine.open() for _ in reqs]
        first = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, plens)])
        steps = [first]
        for j in range(decoded):
            steps.append(engine.step([StepEntry(s, [r[n + j]], [0]) for s, r, n in zip(slots, reqs, plens)]))
        for s in slots:
            engine.close(s)
        stacked = torch.stack(steps, 1)             # [request, step, vocab]
        return [stacked[i] for i in range(len(reqs))]

    times, results = {}, {}
    for name, fn in (("whole", whole), ("one_by_one", one_by_one), ("batched", batched)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        results[name] = fn()
        torch.cuda.synchronize()
        times[name] = round(time.perf_counter() - t0, 2)
    equal = all(torch.equal(a, b) and torch.equal(a, c)
                for a, b, c in zip(results["whole"], results["one_by_one"], results["batched"]))
    finite = all(bool(torch.isfinite(a).all()) for a in results["whole"])
    status = engine.read_status()
    out = {"fp32_cuttings_equal": bool(equal and finite and status == 0), "layers": layers, "prompts": n_prompts,
           "prompt_tokens": sum(plens), "decoded_each": decoded, "rows_compared": n_prompts * (decoded + 1),
           "seconds": times, "build_seconds": round(t_built - t_start, 1),
           "weights_gb": round(engine.memory_plan["weights_bytes"] / 1e9, 1)}
    del engine, results
    gc.collect()
    torch.cuda.empty_cache()
    return out


def decode_timeline(torch, raw, layers, batch, context, prefill_tokens=0):
    """When each kernel of a captured decode step starts and how long it runs (CUPTI through torch.profiler):
    the step as the device sees it, with kernels of the two streams side by side and dependent launches
    resident before their predecessors end.  Prints a table; the times are microseconds from the step's first
    kernel.  ``prefill_tokens`` > 0: the same for the prefill of one prompt of that length (launched kernel
    by kernel from the host, so the gaps between kernels show the host's share)."""
    import numpy as np
    from torch.profiler import ProfilerActivity, profile
    from esp_b200.config import config_from_dict
    from esp_b200.engine import Engine, StepEntry
    from esp_b200.weights import InitSpec

    cfg = config_from_dict(dict(raw, num_hidden_layers=layers))
    engine = Engine.from_random(cfg, seed=0, init=InitSpec(0.02, 0.02, 0.0), dtype="bfloat16",
                                max_tokens=max(batch * (context + 64), prefill_tokens + 64), max_slots=batch + 2)
    rng = np.random.default_rng(1)
    vocab = raw["vocab_size"]
    if prefill_tokens:
        def one():
            s = engine.open()
            engine.step([StepEntry(s, rng.integers(0, vocab, prefill_tokens).tolist(), [prefill_tokens - 1])])
            engine.close(s)
    else:
        slots = [engine.open() for _ in range(batch)]
        for s in slots:
            engine.step([StepEntry(s, rng.integers(0, vocab, context - 26).tolist(), [])])
        temps, tops = [0.0] * batch, [None] * batch

        def one():
            toks = rng.integers(0, vocab, batch).tolist()
            engine.step_and_pick([StepEntry(s, [t], [0]) for s, t in zip(slots, toks)], temps, tops)

    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name),
                    key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(events) if "embed_gather" in e.name]
    step = events[first[-1]:] if first else events
    t0 = step[0].time_range.start
    done = t0
    print(f"{'start':>9} {'runs':>8} {'after the last end':>19}  kernel")
    for e in step:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "")
        print(f"{e.time_range.start - t0:9.1f} {e.time_range.end - e.time_range.start:8.1f} "
              f"{max(0.0, e.time_range.end - max(done, e.time_range.start)):19.1f}  {name[:72]}")
        done = max(done, e.time_range.end)
    print(f"step: {done - t0:.1f} us, {len(step)} kernels, {layers} layers")


def dense_products(torch, raw, tokens=2048):
    """Times the plain dense products of a prefill step (q/k/v, o, shared down) and the fused shared gate/up
    through this library's TMA + tcgen05 kernel (one CTA per tile, and pairs of CTAs) and through cuBLAS."""
    from esp_b200.csrc import ops
    H, nh, nkv, hd, Is = (raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"],
                          raw["shared_expert_intermediate_size"])
    dev = "cuda:0"
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.05).bfloat16()

    def time_us(fn):
        return timed_steps(torch, fn, 3, 20) * 1e3

    rows = []
    for name, n, k in (("q/k/v", (nh + 2 * nkv) * hd, H), ("o", H, nh * hd), ("shared down", H, Is)):
        a, w, c = rnd(tokens, k), rnd(n, k), torch.empty(tokens, n, device=dev)
        flops = 2.0 * tokens * n * k
        own = time_us(lambda: ops.gemm_tc05(a, w, c, st, pair=False))
        pair = time_us(lambda: ops.gemm_tc05(a, w, c, st, pair=True))
        lib = time_us(lambda: torch.mm(a, w.t(), out_dtype=torch.float32, out=c))
        rows.append({"product": name, "n": n, "k": k, "own_us": round(own, 1), "own_pair_us": round(pair, 1),
                     "cublas_us": round(lib, 1), "own_tflops": round(flops / own / 1e6, 1),
                     "cublas_tflops": round(flops / lib / 1e6, 1)})
    a, w, act = rnd(tokens, H), rnd(2 * Is, H), torch.empty(tokens, Is, dtype=torch.bfloat16, device=dev)
    gu = torch.empty(tokens, 2 * Is, device=dev)
    flops = 2.0 * tokens * 2 * Is * H

    def library_then_swiglu():
        torch.mm(a, w.t(), out_dtype=torch.float32, out=gu)
        ops.swiglu(gu, act)

    own = time_us(lambda: ops.gemm_tc05(a, w, act, st, swiglu=True, pair=False))
    pair = time_us(lambda: ops.gemm_tc05(a, w, act, st, swiglu=True, pair=True))
    lib = time_us(library_then_swiglu)
    rows.append({"product": "shared gate/up + SwiGLU", "n": 2 * Is, "k": H, "own_us": round(own, 1),
                 "own_pair_us": round(pair, 1), "cublas_us": round(lib, 1), "own_tflops": round(flops / own / 1e6, 1),
                 "cublas_tflops": round(flops / lib / 1e6, 1)})
    return {"tokens": tokens, "status": int(st.item()), "rows": rows}


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
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="length of the prompt whose prefill is timed")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the 32-bit cuttings check at the headline sizes and the Qwen2-57B-A14B shape")
    ap.add_argument("--timeline", nargs="?", const="decode", choices=["decode", "prefill"], default=None,
                    help="only print when each kernel of one captured decode step (or, with 'prefill', of the prefill "
                         "of --prefill-tokens tokens) starts and ends (default: 2 layers)")
    ap.add_argument("--dense-products", action="store_true",
                    help="only time the dense products of a 2,048-token prefill, own kernel against cuBLAS, and print them")
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

    import torch

    pk = peaks()
    raw, shape_name = SHAPES[a.shape]
    if a.dense_products:
        print(json.dumps({"model": shape_name, **dense_products(torch, raw)}))
        return 0
    if a.timeline:
        decode_timeline(torch, raw, a.layers or 2, a.batch, a.context,
                        a.prefill_tokens if a.timeline == "prefill" else 0)
        return 0
    full_layers = raw["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    clocks = ClockSampler()
    m = measure_shape(torch, raw, a.layers, a.batch, a.context, a.steps, a.warmup, pk,
                      points=() if a.no_points else (1, 64), e2e=not a.no_e2e, prefill=not a.no_prefill, clocks=clocks,
                      prefill_tokens=a.prefill_tokens)

    extras = {}
    if not a.no_extras and a.shape == "a2.7b":
        # BASELINE's other two configurations, each guarded: a failure there must not lose the headline
        try:
            extras["fp32_path"] = fp32_cuttings(torch, raw, a.layers)
        except Exception as e:                                   # noqa: BLE001
            extras["fp32_path"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        try:
            big, big_name = SHAPES["57b-a14b"]
            q = measure_shape(torch, big, big["num_hidden_layers"], a.batch, 8192, max(8, a.steps // 2), a.warmup, pk,
                              points=(1, 64), e2e=False, prefill=True)
            extras["shape_57b_a14b"] = {
                "model": big_name, "layers": big["num_hidden_layers"], "context": 8192,
                "decode_b8": round(q["value"], 1), "decode_b8_ms": round(q["ms_per_step"], 3),
                "decode_b8_hbm_frac": q["roofline"]["frac"], "distinct_b8": round(q["distinct"], 1),
                **q["points"], "points_detail": q["points_detail"], "prefill": q["prefill"]}
        except Exception as e:                                   # noqa: BLE001
            extras["shape_57b_a14b"] = {"error": f"{type(e).__name__}: {e}"[:300]}

    line = {
        "metric": f"decode tok/s at batch {a.batch}", "value": round(m["value"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(m["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
        "impl": "esp_b200",
        "config": {"model": shape_name, "layers": a.layers, "layers_of_model": full_layers,
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "vocab": raw["vocab_size"],
                   "experts": raw["num_experts"], "top_k": raw["num_experts_per_tok"],
                   "moe_intermediate": raw["moe_intermediate_size"],
                   "shared_intermediate": raw["shared_expert_intermediate_size"], "global_batch": a.batch,
                   "seq_len": a.context, "prompt_len": m["prompt_len"], "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (a step reads >10 GB)",
                   "distinct_experts_per_layer": round(m["distinct"], 1)},
        "e2e": m.get("e2e"), "gpu_launches": m["gpu_launches"], "clocks": clocks.summary(), "prefill": m.get("prefill"),
        "roofline": m["roofline"], "points": m["points"], "points_detail": m["points_detail"],
    }
    if "fp32_path" in extras:
        line["fp32_cuttings_equal"] = extras["fp32_path"].get("fp32_cuttings_equal")
    line.update(extras)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
