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


def context(rt, cache, runs, part=None):
    """runs: [(slot, past, new)] -> a StepContext with pages reserved and the index lists ``part`` asks for."""
    from esp_b200.parts.base import StepHost
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
                      want_rows=t([]), block_tables=tables,
                      host={"slots": slots, "news": [n for _, _, n in runs], "pasts": [p for _, p, _ in runs],
                            "starts": list(starts)}, aux={})
    if part is not None:
        host = StepHost(tuple(slots), tuple(n for _, _, n in runs), tuple(p for _, p, _ in runs),
                        tuple(int(v) for v in starts))
        ctx.arrays = {name: t(a) for name, a in part.step_arrays(host).items()}
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
    ctx, growth = context(rt, cache, [(slots[0], 0, cuts[0]), (slots[1], 0, cuts[1])], attn)
    h = torch.cat([xs[0][:cuts[0]], xs[1][:cuts[1]]]).to(dtype).to(DEV)
    y = attn.forward(h, ctx, cache.layers[0]).clone()
    cache.book.commit(growth)
    got[0].append(y[:cuts[0]]), got[1].append(y[cuts[0]:])
    for i in range(20):
        ctx, growth = context(rt, cache, [(slots[0], cuts[0] + i, 1), (slots[1], cuts[1] + i, 1)], attn)
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
    (the sum and the count).  No keys, no values, no pages.

    It may run inside a captured step: it reads nothing from ``ctx.host``; which
    state row a sequence owns comes from ``ctx.seq_slot`` on the device, and the
    runs of rows of a sequence from ``ctx.tok_seq``."""

    graph_safe = True

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
        n, b = h.shape[0], ctx.n_seqs
        seq = ctx.tok_seq.long()                                     # [N] sequence of every row
        slot = ctx.seq_slot.long()                                   # [B] state row of every sequence
        x = h.float()
        # sums of a sequence's rows up to each row: a cumulative sum over all rows minus what came before the sequence
        total = torch.cumsum(x, 0)
        start = ctx.seq_start.long()[:b]                             # first row of every sequence
        before = torch.where(start[:, None] > 0, total[(start - 1).clamp(min=0)], torch.zeros_like(total[:1]))
        state = layer.state[slot]                                    # [B, hidden + 1]
        sums = total - before[seq] + state[seq, :-1]
        counts = (torch.arange(n, device=h.device) - start[seq] + 1).float() + state[seq, -1]
        out = (sums / counts[:, None]) @ self.w.t()
        last = ctx.seq_start.long()[1:b + 1] - 1                     # last row of every sequence
        layer.state.index_copy_(0, slot, torch.cat([sums[last], counts[last, None]], 1))
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


def test_toy_mixer_decodes_from_a_graph_in_another_slot_than_the_one_it_was_captured_in():
    """The graph of a decode step is captured while the sequence sits in one slot and replayed for a
    sequence in another: a part that took its slot from the host when the graph was made would read the
    wrong state on replay."""
    register("mixer", "toy_running_mean", RunningMean)
    eng = Engine.from_random(ToyConfig(), seed=2, init=InitSpec(0.3, 0.0, 0.0), dtype="float32", max_tokens=512)
    assert eng._parts_graph_safe
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(0, 100, 30)]
    s = eng.open()
    whole = eng.step([StepEntry(s, toks, list(range(30)))]).cpu().numpy()
    eng.close(s)

    def prompt_then_decode(slot):
        rows = [eng.step([StepEntry(slot, toks[:6], list(range(6)))]).cpu().numpy()]
        rows += [eng.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in toks[6:]]
        return np.concatenate(rows)

    first = eng.open()
    a = prompt_then_decode(first)                  # eager step, capture, replays: all in this slot
    replays = eng.graph_replays
    assert replays > 10, "the decode steps were meant to replay a captured graph"
    spare = eng.open()                             # holds the slot that ``first`` would get back
    eng.close(first)
    other = eng.open()
    filler = eng.open()
    assert other != first or filler != first
    eng.close(other)
    second = filler                                # a slot that the captured steps never saw
    assert second != first
    b = prompt_then_decode(second)
    assert eng.graph_replays > replays + 10
    eng.close(second), eng.close(spare)
    for got in (a, b):
        assert np.abs(got - whole).max() <= 1e-5 * np.abs(whole).max()


def test_a_part_that_is_not_graph_safe_keeps_the_engine_from_capturing():
    class HostReading(RunningMean):
        graph_safe = False

    register("mixer", "toy_running_mean", HostReading)
    try:
        eng = Engine.from_random(ToyConfig(), seed=2, init=InitSpec(0.3, 0.0, 0.0), dtype="float32", max_tokens=256)
        s = eng.open()
        eng.step([StepEntry(s, [1, 2, 3], [2])])
        for t in range(8):
            eng.step([StepEntry(s, [t], [0])])
        eng.close(s)
        assert eng.graph_replays == 0 and not eng._graphs
    finally:
        register("mixer", "toy_running_mean", RunningMean)


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


# ---------------------------------------------------------------------------
# a toy norm behind a sparse layer, and the model's two ends
# ---------------------------------------------------------------------------
class CenteredNorm(Part):
    """h = (v - mean(v)) / sqrt(var(v) + eps) * weight with v = x + delta: a norm that knows nothing of
    deferred expert sums, so it must be handed plain tensors."""

    graph_safe = True
    seen_delta_types = set()

    def __init__(self, spec, rt):
        self.spec, self.rt, self.weight = spec, rt, None

    def param_specs(self):
        return [ParamSpec(self.spec.weight, (self.spec.width,), "norm_scale")]

    def allocate(self, stored, rt):
        self.weight = torch.empty(self.spec.width, dtype=torch.float32, device=rt.device)
        return {self.spec.weight: self.weight}

    def forward(self, x, delta, h, rows=None, write_x=True, h32=None):
        CenteredNorm.seen_delta_types.add(type(delta))
        v = x if delta is None else x + delta
        if delta is not None and write_x:
            x.copy_(v)
        if rows is not None:
            v = v[rows.long()]
        c = v - v.mean(-1, keepdim=True)
        out = c / torch.sqrt((c * c).mean(-1, keepdim=True) + self.spec.eps) * self.weight
        h.copy_(out)
        if h32 is not None:
            h32.copy_(out)
        return h


def test_a_toy_norm_after_a_sparse_layer_gets_plain_tensors():
    """The sparse block hands on a deferred sum that only the library's own norm folds into its launch;
    a norm from outside must see an ordinary tensor, in the blocks and at the model's end."""
    import dataclasses
    from esp_b200.config import config_from_dict
    from tiny import TINY_A

    class Renormed:
        def __init__(self):
            self.inner = config_from_dict(TINY_A)

        def plan(self):
            plan = self.inner.plan()
            swap = lambda n: dataclasses.replace(n, kind="toy_centered_norm")
            plan.blocks = [dataclasses.replace(b, mixer_norm=swap(b.mixer_norm), ffn_norm=swap(b.ffn_norm))
                           for b in plan.blocks]
            plan.final_norm = swap(plan.final_norm)
            return plan

    register("norm", "toy_centered_norm", CenteredNorm)
    CenteredNorm.seen_delta_types = set()
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(Renormed(), seed=6, init=InitSpec(0.05, 0.02, 0.01), dtype=dtype, max_tokens=256)
        toks = [int(t) for t in np.random.default_rng(2).integers(0, 256, 50)]
        s = eng.open()
        whole = eng.step([StepEntry(s, toks, list(range(50)))]).cpu().numpy()
        eng.close(s)
        s = eng.open()
        rows = [eng.step([StepEntry(s, toks[:20], list(range(20)))]).cpu().numpy()]
        rows += [eng.step([StepEntry(s, [t], [0])]).cpu().numpy() for t in toks[20:]]
        eng.close(s)
        assert np.isfinite(whole).all() and eng.read_status() == 0
        tol = 1e-5 if dtype == "float32" else 4 * 2.0 ** -8
        assert np.abs(np.concatenate(rows) - whole).max() <= tol * np.abs(whole).max()
    assert CenteredNorm.seen_delta_types <= {torch.Tensor, type(None)}, CenteredNorm.seen_delta_types


def test_embedding_scale_and_logit_softcap_of_a_plan():
    """The model's two ends take a scale and a cap from the plan: the scaled model equals the unscaled one
    whose table was multiplied beforehand, and the cap is cap * tanh(logits / cap)."""
    scale, cap = 3.0, 0.25

    class Ends(ToyAttentionConfig):
        def __init__(self, with_ends):
            self.with_ends = with_ends

        def plan(self):
            plan = super().plan()
            plan.head_weight = "t.head.weight"
            if self.with_ends:
                plan.embed_scale, plan.logit_softcap = scale, cap
            return plan

    register("position", "toy_scaled_position", ScaledPosition)
    register("ffn", "toy_top1_ffn", Top1Ffn)
    toks = [int(t) for t in np.random.default_rng(4).integers(0, 90, 25)]
    outs = []
    for with_ends in (False, True):
        eng = Engine.from_random(Ends(with_ends), seed=3, init=InitSpec(0.2, 0.05, 0.0), dtype="float32", max_tokens=256)
        if not with_ends:
            eng.model.embed.mul_(scale)
        s = eng.open()
        outs.append(eng.step([StepEntry(s, toks, list(range(25)))]).cpu().numpy())
        eng.close(s)
        assert eng.read_status() == 0
    want = cap * np.tanh(outs[0].astype(np.float64) / cap)
    assert np.abs(outs[0]).max() > cap, "the cap is meant to bite"
    assert np.abs(outs[1] - want).max() <= 2e-6 * cap


# ---------------------------------------------------------------------------
# two probes of the attention part (crates/esp/src/infer/decoder/attention.rs:518-627)
# ---------------------------------------------------------------------------
def run_attention(attn, rt, dtype, x, cut):
    """The part's output for the rows of ``x``: the first ``cut`` rows as one step, the rest one by one."""
    cache = Cache([(attn.kv_layout(), None, None)], 1024, 2, 600, dtype, rt.device)
    slot = cache.open()
    outs = []
    for a, b in [(0, cut)] + [(i, i + 1) for i in range(cut, x.shape[0])]:
        ctx, growth = context(rt, cache, [(slot, a, b - a)], attn)
        outs.append(attn.forward(x[a:b].to(dtype).to(DEV), ctx, cache.layers[0]).clone())
        cache.book.commit(growth)
    assert rt.status.item() == 0
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd, rows, cut", [(24, 40, 33), (128, 200, 200), (128, 150, 140), (64, 70, 64)])
def test_changing_the_last_token_changes_no_earlier_row(dtype, hd, rows, cut):
    """The causal-mask probe: with only the last token moved, every earlier row's output keeps its bits (a
    missing or inverted mask, or a kernel whose rows share a reduction, would show), and the last row's
    output changes."""
    hidden = 96
    spec = AttentionSpec(hidden, 4, 2, hd, True, False, None, PositionSpec("rope_split_half", hd, 1e4, 600), "a.")
    rt, attn, _w = make("mixer", spec, dtype)
    x = torch.randn(rows, hidden, generator=torch.Generator().manual_seed(5)) * 0.5
    moved = x.clone()
    moved[-1] += 1.0
    a, b = run_attention(attn, rt, dtype, x, cut), run_attention(attn, rt, dtype, moved, cut)
    assert torch.equal(a[:-1], b[:-1]), "an earlier position changed when only the last token moved"
    assert (a[-1] - b[-1]).abs().max() > 1e-3, "the moved position itself must change"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd, rows, cut", [(24, 40, 33), (128, 200, 190), (64, 140, 130)])
def test_grouped_heads_equal_full_heads_with_duplicated_key_value_blocks(dtype, hd, rows, cut):
    """Attention with 2 key/value heads for 4 query heads equals attention with 4 key/value heads whose k and
    v weights (and biases) repeat each block once per group: query head i reads key/value head i // 2."""
    hidden, nh, nkv = 96, 4, 2
    pos = PositionSpec("rope_split_half", hd, 1e4, 600)
    rt, gqa, _w = make("mixer", AttentionSpec(hidden, nh, nkv, hd, True, False, None, pos, "a."), dtype)
    rt2, mha, _w2 = make("mixer", AttentionSpec(hidden, nh, nh, hd, True, False, None, pos, "a."), dtype, seed=8)
    q_rows, kv_rows = nh * hd, nkv * hd
    dup = lambda t: t.reshape(nkv, hd, *t.shape[1:]).repeat_interleave(nh // nkv, 0).reshape(nh * hd, *t.shape[1:])
    for src, dst in ((gqa.w_qkv, mha.w_qkv), (gqa.b_qkv, mha.b_qkv)):
        dst[:q_rows].copy_(src[:q_rows])
        dst[q_rows:q_rows + nh * hd].copy_(dup(src[q_rows:q_rows + kv_rows]))
        dst[q_rows + nh * hd:].copy_(dup(src[q_rows + kv_rows:]))
    mha.w_o.copy_(gqa.w_o)
    x = torch.randn(rows, hidden, generator=torch.Generator().manual_seed(6)) * 0.5
    a, b = run_attention(gqa, rt, dtype, x, cut), run_attention(mha, rt2, dtype, x, cut)
    assert torch.equal(a, b), f"grouped and duplicated heads differ by {(a - b).abs().max().item():.3e}"
