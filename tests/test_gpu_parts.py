"""Each part of a layer alone (norm, position encoding with the cache write,
attention, dense feed-forward, sparse feed-forward, block), built from a spec
through the registries with its own sizes, against the plain functions; and a
toy mixer with state of its own, defined here, that is registered, built and
stepped without any change to the library."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from esp_b200.cache import Cache, KvLayout, StateSpec
from esp_b200.config.plan import (AttentionSpec, BlockSpec, DenseFfnSpec, ModelPlan, MoeFfnSpec, NormSpec,
                                  PositionSpec, ScheduleEntry)
from esp_b200.engine import Engine, StepEntry
from esp_b200.parts import ParamSpec, Part, Runtime, StepContext, build, register
from esp_b200.weights import InitSpec, RandomSource, load_into

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 4 * 2.0 ** -8}


def make(family, spec, dtype, seed=3, init=InitSpec(0.08, 0.05, 0.05)):
    rt = Runtime(DEV, dtype)
    part = build(family, spec, rt)
    from esp_b200.parts import walk
    specs = [s for p in walk(part) for s in p.param_specs()]
    src = RandomSource(specs, seed, init, dtype)
    load_into(part, src, rt, ())
    weights = {n: src.host_tensor(n).float().numpy() for n in src.names()}
    return rt, part, weights


def context(rt, cache, runs):
    """runs: [(slot, past, new)] -> a StepContext with pages reserved."""
    growth = {s: n for s, _p, n in runs}
    cache.book.reserve(growth)
    slots = [s for s, _, _ in runs]
    seq = np.repeat(np.arange(len(runs)), [n for _, _, n in runs]).astype(np.int32)
    pos = np.concatenate([np.arange(p, p + n) for _, p, n in runs]).astype(np.int32)
    starts = np.concatenate([[0], np.cumsum([n for _, _, n in runs])]).astype(np.int32)
    stride = cache.max_table_stride(slots, growth)
    t = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    tables = [t(g.table_rows(slots, stride)) for g in cache.book.groups]
    ctx = StepContext(n_tokens=len(seq), n_seqs=len(runs), max_new=max(n for _, _, n in runs),
                      max_len=max(p + n for _, p, n in runs), tok_ids=t(np.zeros(len(seq))), tok_seq=t(seq),
                      tok_pos=t(pos), seq_slot=t(slots), seq_start=t(starts), seq_past=t([p for _, p, _ in runs]),
                      want_rows=t([]), q_tile_seq=t([i for i, (_s, _p, n) in enumerate(runs) for _ in range(0, n, 64)]),
                      q_tile_first=t([f for _s, _p, n in runs for f in range(0, n, 64)]), block_tables=tables,
                      host={"slots": slots, "news": [n for _, _, n in runs], "pasts": [p for _, p, _ in runs],
                            "starts": list(starts)}, aux={})
    return ctx, growth


def assert_close(got, ref, dtype, what):
    got = got.float().cpu().numpy()
    scale = max(1e-9, np.abs(ref).max())
    err = np.abs(got - ref).max()
    assert err <= TOL[dtype] * scale, f"{what}: {err:.3e} > {TOL[dtype] * scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    rt, norm, w = make("norm", NormSpec("rmsnorm", 200, 3e-4, "n.weight"), dtype)
    x = torch.randn(7, 200, device=DEV)
    d = torch.randn(7, 200, device=DEV)
    h = torch.empty(7, 200, dtype=dtype, device=DEV)
    ref = plain.rms_norm((x + d).cpu().numpy(), w["n.weight"], 3e-4)
    norm.forward(x, d, h)
    assert_close(h, ref, dtype, "rmsnorm part")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd, window, theta", [(6, 3, 40, None, 5e5), (4, 1, 64, 9, 1e4)])
def test_attention_part_with_cache_across_steps(dtype, nh, nkv, hd, window, theta):
    hidden = 88
    spec = AttentionSpec(hidden, nh, nkv, hd, True, False, window, PositionSpec("rope_split_half", hd, theta, 300), "a.")
    rt, attn, w = make("mixer", spec, dtype)
    cache = Cache([(attn.kv_layout(), None, None)], 1024, 4, 300, dtype, rt.device)
    lens = [150, 70]
    xs = [torch.randn(n, hidden) * 0.5 for n in lens]
    c = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rope_theta": theta}
    refs = [plain.attention(c, w, "a.", x.to(dtype).float().numpy(), window) for x in xs]
    slots = [cache.open(), cache.open()]
    got = [[], []]
    # both sequences start together with unequal prompts, then go on one token at a time
    cuts = [lens[0] - 20, lens[1] - 20]
    ctx, growth = context(rt, cache, [(slots[0], 0, cuts[0]), (slots[1], 0, cuts[1])])
    h = torch.cat([xs[0][:cuts[0]], xs[1][:cuts[1]]]).to(dtype).to(DEV)
    y = attn.forward(h, ctx, cache.layers[0]).clone()
    cache.book.commit(growth)
    got[0].append(y[:cuts[0]]), got[1].append(y[cuts[0]:])
    for i in range(20):
        ctx, growth = context(rt, cache, [(slots[0], cuts[0] + i, 1), (slots[1], cuts[1] + i, 1)])
        h = torch.stack([xs[0][cuts[0] + i], xs[1][cuts[1] + i]]).to(dtype).to(DEV)
        y = attn.forward(h, ctx, cache.layers[0]).clone()
        cache.book.commit(growth)
        got[0].append(y[:1]), got[1].append(y[1:])
    assert rt.status.item() == 0
    for s in range(2):
        assert_close(torch.cat(got[s]), refs[s], dtype, f"attention part, sequence {s}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_ffn_part(dtype):
    rt, ffn, w = make("ffn", DenseFfnSpec(72, 200, "m."), dtype)
    h = (torch.randn(19, 72) * 0.5).to(dtype)
    y = ffn.forward(h.to(DEV), None)
    assert_close(y, plain.dense_mlp(w, "m.", h.float().numpy()), dtype, "dense feed-forward part")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm_topk", [False, True])
def test_moe_ffn_part(dtype, norm_topk):
    spec = MoeFfnSpec(72, 7, 3, norm_topk, 40, 56, "m.")
    rt, ffn, w = make("ffn", spec, dtype, init=InitSpec(0.15, 0.0, 0.0))
    rt.record_routing = True
    h32 = torch.randn(33, 72) * 0.5
    h = h32.to(dtype)
    ctx = type("Ctx", (), {"aux": {}})()
    y = ffn.forward(h.to(DEV), ctx, h32=h32.to(DEV) if dtype != torch.float32 else None)
    if hasattr(y, "materialize"):          # the block may leave its ordered sum to the norm that follows
        y = y.materialize()
    c = {"num_experts_per_tok": 3, "norm_topk_prob": norm_topk}
    (_prefix, _row0, ids, _wts, _probs), = ctx.aux["routing"]
    # the plain block routes from the same unrounded rows and computes from the rounded ones
    rec = []
    ids_plain, p = plain.route(c, w, "m.", h32.numpy())
    assert np.array_equal(np.sort(ids.cpu().numpy(), 1), np.sort(ids_plain, 1))
    ref = plain_moe_with_router_input(c, w, "m.", h.float().numpy(), h32.numpy())
    assert_close(y, ref, dtype, "sparse feed-forward part")
    assert rt.status.item() == 0


def plain_moe_with_router_input(c, w, prefix, x, router_x):
    """plain.moe_block with the routing probabilities taken from ``router_x``."""
    ids, p = plain.route(c, w, prefix, router_x)
    w2 = dict(w)
    out = np.zeros_like(x)
    chosen = np.zeros(p.shape, dtype=bool)
    np.put_along_axis(chosen, ids, True, axis=-1)
    s = np.where(chosen, p, 0).sum(-1) if c["norm_topk_prob"] else np.ones(p.shape[0], np.float32)
    for e in range(p.shape[1]):
        rows = np.nonzero(chosen[:, e])[0]
        if rows.size:
            ep = f"{prefix}experts.{e}."
            y = plain.swiglu(x[rows], w[ep + "gate_proj.weight"], w[ep + "up_proj.weight"], w[ep + "down_proj.weight"])
            out[rows] += y * (p[rows, e] / s[rows])[:, None]
    sp = prefix + "shared_expert."
    shared = plain.swiglu(x, w[sp + "gate_proj.weight"], w[sp + "up_proj.weight"], w[sp + "down_proj.weight"])
    gate = 1.0 / (1.0 + np.exp(-(router_x @ w[prefix + "shared_expert_gate.weight"].T)))
    return out + gate * shared


# ---------------------------------------------------------------------------
# a toy mixer with state of its own
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    prefix: str
    kind: str = "toy_running_mean"


class RunningMean(Part):
    """delta_t = W * mean(h_0 .. h_t): needs the sum of the sequence's earlier
    rows, which it keeps as per-sequence state of fixed size [hidden + 1]
    (the sum and the count).  No keys, no values, no pages."""

    def __init__(self, spec, rt):
        self.spec, self.rt, self.w = spec, rt, None

    def param_specs(self):
        return [ParamSpec(self.spec.prefix + "mix.weight", (self.spec.hidden, self.spec.hidden), "matrix")]

    def allocate(self, stored, rt):
        self.w = torch.empty(self.spec.hidden, self.spec.hidden, dtype=torch.float32, device=rt.device)
        return {self.spec.prefix + "mix.weight": self.w}

    def kv_layout(self):
        return None

    def state_spec(self):
        return StateSpec((self.spec.hidden + 1,), torch.float32)

    def forward(self, h, ctx, layer):
        out = torch.empty(h.shape[0], self.spec.hidden, dtype=torch.float32, device=h.device)
        for b, slot in enumerate(ctx.host["slots"]):
            a, e = ctx.host["starts"][b], ctx.host["starts"][b + 1]
            state = layer.state[slot]
            sums = state[:-1] + torch.cumsum(h[a:e].float(), 0)
            counts = state[-1] + torch.arange(1, e - a + 1, device=h.device, dtype=torch.float32)
            out[a:e] = (sums / counts[:, None]) @ self.w.t()
            state[:-1] = sums[-1]
            state[-1] = counts[-1]
        return out


class ToyConfig:
    """Stands where an architecture's configuration stands: it only has to give a plan."""

    def __init__(self, hidden=48, vocab=100, layers=2):
        self.hidden, self.vocab, self.layers = hidden, vocab, layers

    def plan(self):
        blocks = []
        for i in range(self.layers):
            p = f"toy.{i}."
            blocks.append(BlockSpec(RunningMeanSpec(self.hidden, p), DenseFfnSpec(self.hidden, 64, p + "mlp."),
                                    NormSpec("rmsnorm", self.hidden, 1e-6, p + "n1.weight"),
                                    NormSpec("rmsnorm", self.hidden, 1e-6, p + "n2.weight")))
        return ModelPlan("ToyRunningMean", self.hidden, self.vocab, 512, blocks,
                         [ScheduleEntry(i) for i in range(self.layers)],
                         NormSpec("rmsnorm", self.hidden, 1e-6, "toy.norm.weight"), "toy.embed.weight", None)


def test_toy_mixer_with_its_own_state_runs_through_the_engine():
    register("mixer", "toy_running_mean", RunningMean)
    eng = Engine.from_random(ToyConfig(), seed=2, init=InitSpec(0.3, 0.0, 0.0), dtype="float32", max_tokens=512)
    assert not eng.cache.book.groups, "a model without attention needs no key/value pools"
    rng = np.random.default_rng(0)
    toks = [int(t) for t in rng.integers(0, 100, 40)]
    other = [int(t) for t in rng.integers(0, 100, 13)]
    # whole
    s = eng.open()
    whole = eng.step([StepEntry(s, toks, list(range(40)))]).cpu().numpy()
    eng.close(s)
    # the slot is used again: its state must start from zero; cut in three runs, beside another sequence
    s, o = eng.open(), eng.open()
    parts = [eng.step([StepEntry(s, toks[:9], list(range(9))), StepEntry(o, other[:5], [])]).cpu().numpy()]
    parts.append(eng.step([StepEntry(o, other[5:], []), StepEntry(s, toks[9:30], list(range(21)))]).cpu().numpy())
    for t in toks[30:]:
        parts.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy())
    eng.close(s), eng.close(o)
    cut = np.concatenate(parts)
    assert np.abs(cut - whole).max() <= 1e-5 * np.abs(whole).max()
    # and the plain restatement of the toy
    names = {sp.name: sp for p in eng.model.all_parts() for sp in p.param_specs() if not sp.optional}
    w = {n: eng_tensor(eng, n) for n in names}
    x = w["toy.embed.weight"][toks]
    for i in range(2):
        p = f"toy.{i}."
        h = plain.rms_norm(x, w[p + "n1.weight"], 1e-6)
        x = x + (np.cumsum(h, 0) / np.arange(1, 41)[:, None]) @ w[p + "mix.weight"].T
        h = plain.rms_norm(x, w[p + "n2.weight"], 1e-6)
        x = x + plain.dense_mlp(w, p + "mlp.", h)
    ref = plain.rms_norm(x, w["toy.norm.weight"], 1e-6) @ w["toy.embed.weight"].T
    assert np.abs(whole - ref).max() <= 2e-5 * np.abs(ref).max()


def eng_tensor(eng, name):
    from esp_b200.weights.random_init import RandomSource
    specs = [sp for p in eng.model.all_parts() for sp in p.param_specs()]
    return RandomSource(specs, 2, InitSpec(0.3, 0.0, 0.0), torch.float32).host_tensor(name).numpy()


def test_schedule_may_run_a_layer_twice_and_share_a_cache(tmp_path):
    """The order of layers is data: here layer 0 runs, then layer 1, then
    layer 0 again reading the keys and values its first call stored."""
    from esp_b200.config import config_from_dict
    from tiny import TINY_A

    class Looped:
        def __init__(self):
            self.inner = config_from_dict(TINY_A)

        def plan(self):
            plan = self.inner.plan()
            plan.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)]
            return plan

    eng = Engine.from_random(Looped(), seed=4, init=InitSpec(0.05, 0.02, 0.01), dtype="float32", max_tokens=256)
    assert len(eng.cache.layers) == 3 and eng.cache.layers[2].k.data_ptr() == eng.cache.layers[0].k.data_ptr()
    assert eng.cache.layers[2].writes is False and eng.cache.k_pools[0].shape[0] == 2
    toks = list(range(3, 30))
    s = eng.open()
    whole = eng.step([StepEntry(s, toks, list(range(len(toks))))]).cpu().numpy()
    eng.close(s)
    s = eng.open()
    rows = [eng.step([StepEntry(s, toks[:10], list(range(10)))]).cpu().numpy()]
    rows += [eng.step([StepEntry(s, [t], [0])]).cpu().numpy() for t in toks[10:]]
    eng.close(s)
    assert np.array_equal(np.concatenate(rows), whole)
    assert np.isfinite(whole).all() and eng.read_status() == 0


# ---------------------------------------------------------------------------
# a toy position encoding and a toy routed feed-forward, both defined here
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class ScaledPositionSpec:
    """Queries and keys of position p are multiplied by 1 + slope * p (a made-up encoding)."""
    slope: float
    kind: str = "toy_scaled_position"


class ScaledPosition(Part):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt

    def rotate_and_store(self, qkv, bias, ctx, q_out, layer, nh, nkv, hd, status):
        from esp_b200.csrc import ops
        scale = 1.0 + self.spec.slope * ctx.tok_pos.float()
        if bias is not None:
            qkv.add_(bias)
        qkv[:, :(nh + nkv) * hd].mul_(scale[:, None])
        table = ctx.block_tables[layer.group]
        ops.rope_kvwrite(qkv, None, ctx.tok_seq, ctx.tok_pos, None, None, 0, q_out, layer.k, layer.v, table, layer.page,
                         nh, nkv, hd, layer.writes, status)


@dataclass(frozen=True)
class Top1FfnSpec:
    hidden: int
    choices: int
    inner: int
    prefix: str
    kind: str = "toy_top1_ffn"


class Top1Ffn(Part):
    """Each token goes to the one of ``choices`` small MLPs whose key has the largest dot product with it."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.keys = self.w_in = self.w_out = None

    def param_specs(self):
        s, p = self.spec, self.spec.prefix
        return [ParamSpec(p + "keys", (s.choices, s.hidden), "matrix"),
                ParamSpec(p + "w_in", (s.choices * s.inner, s.hidden), "matrix"),
                ParamSpec(p + "w_out", (s.choices * s.hidden, s.inner), "matrix")]

    def allocate(self, stored, rt):
        s, p, f32 = self.spec, self.spec.prefix, dict(dtype=torch.float32, device=rt.device)
        self.keys = torch.empty(s.choices, s.hidden, **f32)
        self.w_in = torch.empty(s.choices * s.inner, s.hidden, **f32)
        self.w_out = torch.empty(s.choices * s.hidden, s.inner, **f32)
        return {p + "keys": self.keys, p + "w_in": self.w_in, p + "w_out": self.w_out}

    def forward(self, h, ctx, h32=None):
        s = self.spec
        x = h.float()
        choice = (x @ self.keys.t()).argmax(-1)
        out = torch.zeros(x.shape[0], s.hidden, device=x.device)
        for c in range(s.choices):
            rows = (choice == c).nonzero()[:, 0]
            if rows.numel():
                w_in, w_out = self.w_in[c * s.inner:(c + 1) * s.inner], self.w_out[c * s.hidden:(c + 1) * s.hidden]
                out[rows] = torch.relu(x[rows] @ w_in.t()) @ w_out.t()
        return out


class ToyAttentionConfig:
    """Attention with the toy position encoding, the toy routed feed-forward, two layers."""

    def plan(self):
        hidden, blocks = 64, []
        for i in range(2):
            p = f"t.{i}."
            mixer = AttentionSpec(hidden, 4, 2, 16, True, False, None, ScaledPositionSpec(0.01), p + "attn.")
            blocks.append(BlockSpec(mixer, Top1FfnSpec(hidden, 3, 40, p + "ffn."),
                                    NormSpec("rmsnorm", hidden, 1e-6, p + "n1.weight"),
                                    NormSpec("rmsnorm", hidden, 1e-6, p + "n2.weight")))
        return ModelPlan("ToyScaledTop1", hidden, 90, 256, blocks, [ScheduleEntry(0), ScheduleEntry(1)],
                         NormSpec("rmsnorm", hidden, 1e-6, "t.norm.weight"), "t.embed.weight", None)


def test_toy_position_encoding_and_toy_routed_ffn_run_through_the_engine():
    """Parts of two more families, registered from outside: another position encoding (used by the library's
    own attention) and a feed-forward with routing of its own; whole prompt equals token by token."""
    register("position", "toy_scaled_position", ScaledPosition)
    register("ffn", "toy_top1_ffn", Top1Ffn)
    eng = Engine.from_random(ToyAttentionConfig(), seed=3, init=InitSpec(0.2, 0.05, 0.0), dtype="float32", max_tokens=512)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, 90, 70)]
    s = eng.open()
    whole = eng.step([StepEntry(s, toks, list(range(70)))]).cpu().numpy()
    eng.close(s)
    s = eng.open()
    rows = [eng.step([StepEntry(s, toks[:33], list(range(33)))]).cpu().numpy()]
    rows += [eng.step([StepEntry(s, [t], [0])]).cpu().numpy() for t in toks[33:]]
    eng.close(s)
    cut = np.concatenate(rows)
    assert np.isfinite(whole).all() and eng.read_status() == 0
    assert np.abs(cut - whole).max() <= 1e-5 * np.abs(whole).max()
    # the encoding is felt: the same token at another position gives other logits
    s = eng.open()
    a = eng.step([StepEntry(s, [5, 7, 7], [1, 2])]).cpu().numpy()
    eng.close(s)
    assert np.abs(a[0] - a[1]).max() > 1e-4
