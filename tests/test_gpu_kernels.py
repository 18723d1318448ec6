"""Each kernel alone against a plain PyTorch reference of the same operation in
float32/float64, at sizes other than the models' (widths and vocabularies that
are no power of two, odd row counts, empty groups), with inputs made so that a
fault shows: one score that stands out at a far key, at the window's edge, at
a page boundary, in another sequence's pages."""
import numpy as np
import pytest
import torch

import plain_qwen2_moe as plain
from esp_b200.csrc import ops
from esp_b200.weights.random_init import normal_values

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, ref, dtype, what="", k=None):
    """``k``: length of the sums behind a tensor-core product.  Products of bfloat16 values are exact in
    float; the tensor cores add them into a float accumulator 16 at a time and may truncate, so the
    error is bounded by one float ulp (2^-24 relative) of the running sum per step of 16."""
    got, ref = got.double().cpu(), ref.double().cpu()
    tol = 2e-6 if dtype == torch.float32 else 2.0 ** -7
    if k is not None and dtype == torch.float32:
        tol = max(tol, (k / 16) * 2.0 ** -24)
    scale = max(1e-9, float(ref.abs().max()))
    err = float((got - ref).abs().max())
    assert err <= tol * scale, f"{what}: max error {err:.3e} on scale {scale:.3e} (bound {tol * scale:.3e})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(dtype):
    table = rnd(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32, device=DEV)
    x = torch.empty(5, 200, device=DEV)
    st = status()
    ops.embed_gather(table, ids, x, st)
    assert torch.equal(x, table.float()[ids.long()]) and st.item() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [200, 2072])
def test_add_rmsnorm(dtype, width):
    x = rnd(9, width)
    y = rnd(9, width, seed=1)
    gamma = 1 + 0.1 * rnd(width, seed=2)
    eps = 1e-5
    ref_x = x + y
    ref = ref_x.double() / torch.sqrt((ref_x.double() ** 2).mean(-1, keepdim=True) + eps) * gamma.double()
    x1, h, h32 = x.clone(), torch.empty(9, width, dtype=dtype, device=DEV), torch.empty(9, width, device=DEV)
    ops.add_rmsnorm(x1, y, gamma, h, eps, h32=h32)
    assert torch.equal(x1, ref_x)
    close(h, ref, dtype, "normed rows")
    close(h32, ref, torch.float32, "unrounded rows")
    # selected rows, residual left alone
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    x2, h2 = x.clone(), torch.empty(3, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(x2, y, gamma, h2, eps, rows=rows, write_x=False)
    assert torch.equal(x2, x)
    close(h2, ref[rows.long()], dtype, "selected rows")
    # no addend
    x3, h3 = x.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(x3, None, gamma, h3, eps)
    close(h3, x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * gamma.double(), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    gu = rnd(13, 2 * 37, scale=3.0)
    act = torch.empty(13, 37, dtype=dtype, device=DEV)
    ops.swiglu(gu, act)
    g, u = gu[:, :37].double(), gu[:, 37:].double()
    close(act, g / (1 + torch.exp(-g)) * u, dtype)


@pytest.mark.parametrize("a_dt, w_dt, c_dt", [(torch.float32, torch.float32, torch.float32),
                                               (torch.bfloat16, torch.bfloat16, torch.float32),
                                               (torch.bfloat16, torch.float32, torch.float32),
                                               (torch.float32, torch.bfloat16, torch.bfloat16)])
def test_gemm_simt_dense(a_dt, w_dt, c_dt):
    m, n, k = 77, 130, 150
    a, w = rnd(m, k, dtype=a_dt), rnd(n, k, dtype=w_dt, seed=1)
    bias, scale = rnd(n, seed=2), rnd(m, seed=3)
    c = torch.empty(m, n, dtype=c_dt, device=DEV)
    ops.gemm_simt(a, w, c, bias=bias, row_scale=scale)
    ref = (a.double() @ w.double().t() + bias.double()) * scale.double()[:, None]
    close(c, ref, c_dt, "dense")
    # a single row gives the same bits as that row inside the larger product
    c1 = torch.empty(1, n, dtype=c_dt, device=DEV)
    ops.gemm_simt(a[5:6], w, c1, bias=bias, row_scale=scale[5:6].contiguous())
    assert torch.equal(c1[0], c[5])


def test_gemm_simt_grouped_with_gather_and_empty_groups():
    g, n, k = 5, 70, 90
    counts = [3, 0, 66, 1, 0]
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    total = sum(counts)
    src = rnd(40, k)
    a_rows = torch.tensor(np.random.default_rng(0).integers(0, 40, total), dtype=torch.int32, device=DEV)
    w = rnd(g, n, k, seed=1)
    scale = rnd(total, seed=2)
    c = torch.full((total + 3, n), 7.0, device=DEV)
    ops.gemm_simt(src, w, c, a_rows=a_rows, row_scale=scale, group_offsets=offsets, rows=total)
    row = 0
    for e, cnt in enumerate(counts):
        for _ in range(cnt):
            ref = (src[a_rows[row].long()].double() @ w[e].double().t()) * scale[row].double()
            close(c[row], ref, torch.float32, f"group {e} row {row}")
            row += 1
    assert torch.all(c[total:] == 7.0), "rows beyond the groups were written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd, rot", [(24, 24), (128, 128), (40, 16)])
def test_rope_kvwrite(dtype, hd, rot):
    nh, nkv, page, n_pages = 3, 1, 64, 6
    # two sequences: 70 new tokens from position 60, and one token at position 129
    pos = list(range(60, 130)) + [129]
    seq = [0] * 70 + [1]
    n = len(pos)
    table = torch.tensor([[4, 0, 2], [1, 5, 3]], dtype=torch.int32, device=DEV)
    qkv = rnd(n, (nh + 2 * nkv) * hd)
    bias = rnd((nh + 2 * nkv) * hd, seed=5)
    theta = 10000.0
    cos_np, sin_np = plain.rope_angles(np.arange(200), rot, theta)
    cos, sin = torch.from_numpy(cos_np).to(DEV), torch.from_numpy(sin_np).to(DEV)
    q_out = torch.empty(n, nh * hd, dtype=dtype, device=DEV)
    kc = torch.zeros(n_pages, nkv, page, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    st = status()
    ops.rope_kvwrite(qkv, bias, torch.tensor(seq, dtype=torch.int32, device=DEV),
                     torch.tensor(pos, dtype=torch.int32, device=DEV), cos, sin, rot, q_out, kc, vc, table, page,
                     nh, nkv, hd, True, st)
    assert st.item() == 0
    x = (qkv + bias).cpu().numpy().reshape(n, nh + 2 * nkv, hd)
    rotated = x.copy()
    rotated[:, :nh + nkv, :rot] = plain.apply_rope(x[:, :nh + nkv, :rot], cos_np[pos], sin_np[pos])
    close(q_out.view(n, nh, hd), torch.from_numpy(rotated[:, :nh]), dtype, "queries")
    tbl = table.cpu().numpy()
    for i in range(n):
        pg = tbl[seq[i], pos[i] // page]
        close(kc[pg, 0, pos[i] % page], torch.from_numpy(rotated[i, nh]), dtype, f"key of token {i}")
        close(vc[pg, 0, pos[i] % page], torch.from_numpy(x[i, nh + 1]), dtype, f"value of token {i}")
    written = {(tbl[seq[i], pos[i] // page], pos[i] % page) for i in range(n)}
    mask = torch.ones(n_pages, page, dtype=torch.bool)
    for pg, ip in written:
        mask[pg, ip] = False
    assert torch.all(kc[:, 0][mask.to(DEV)] == 0), "a cache row that no token owns was written"


def paged(seqs_k, seqs_v, tables, n_pages, nkv, hd, dtype, page=64):
    kc = torch.zeros(n_pages, nkv, page, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    for s, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for p in range(k.shape[0]):
            pg = tables[s][p // page]
            kc[pg, :, p % page] = k[p].to(dtype)
            vc[pg, :, p % page] = v[p].to(dtype)
    return kc, vc


def attention_reference(q, k, v, pos, window, group):
    """q [nh, hd] at absolute position pos over k, v [len, nkv, hd] in float64."""
    nh, hd = q.shape
    out = torch.zeros(nh, hd, dtype=torch.float64)
    lo = 0 if not window else max(0, pos - window + 1)
    for h in range(nh):
        kk, vv = k[lo:pos + 1, h // group].double(), v[lo:pos + 1, h // group].double()
        s = (kk @ q[h].double()) / np.sqrt(hd)
        out[h] = torch.softmax(s, 0) @ vv
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd, window", [(6, 2, 40, None), (4, 1, 128, 100), (2, 2, 256, None), (8, 4, 16, 65)])
def test_attention_finds_the_key_that_matters(dtype, nh, nkv, hd, window):
    """Three sequences in interleaved pages.  In each, one key is made to carry
    almost all of a query's weight: a far key among hundreds, the oldest key a
    window still shows, the key just outside it, keys on both sides of a page
    boundary.  Dropping, shifting or misplacing any of them changes the output
    by far more than rounding."""
    torch.manual_seed(1)
    lens = [700, 130, 65]
    group = nh // nkv
    tables = [[3 * i + s for i in range(12)] for s in range(3)]        # interleaved pages
    ks = [torch.randn(n, nkv, hd) * 0.3 for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    queries = []   # (sequence, position, target key)
    last = lens[0] - 1
    w = window or 10 ** 9
    for target in {3, 63, 64, 65, 127, 128, max(0, last - w + 1), max(0, last - w), last}:
        queries.append((0, last, target))
    queries += [(1, 129, 64), (1, 100, 0), (2, 64, 63), (2, 0, 0), (2, 1, 0)]
    q = torch.randn(len(queries), nh, hd) * 0.3
    for i, (s, p, target) in enumerate(queries):
        for h in range(nh):
            # align the query with the target key and give the pair a large norm
            ks[s][target, h // group] = ks[s][target, h // group] / ks[s][target, h // group].norm() * 6.0
            q[i, h] = ks[s][target, h // group] * (np.sqrt(hd) * 3.0 / 6.0)
    # (a later query may re-scale an earlier target; keys are final now, so references below are consistent)
    qd = q.to(dtype)
    kc, vc = paged(ks, vs, tables, 36, nkv, hd, dtype)
    table = torch.tensor([t + [-1] * 0 for t in tables], dtype=torch.int32, device=DEV)
    out = torch.empty(len(queries), nh * hd, dtype=dtype, device=DEV)
    st = status()
    ops.attn_simt(qd.reshape(len(queries), nh * hd).to(DEV), kc, vc, out,
                  torch.tensor([s for s, _, _ in queries], dtype=torch.int32, device=DEV),
                  torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=DEV), table, 64, nh, nkv, hd,
                  window, st)
    assert st.item() == 0
    for i, (s, p, target) in enumerate(queries):
        ref = attention_reference(qd[i].float(), ks[s].to(dtype).float(), vs[s].to(dtype).float(), p, window, group)
        close(out[i].view(nh, hd), ref, dtype, f"query {i} (sequence {s}, position {p}, target key {target})")


@pytest.mark.parametrize("h_dt, w_dt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("norm", [False, True])
def test_router_topk(h_dt, w_dt, norm):
    n, width, e, k = 11, 150, 10, 3
    h = rnd(n, width, dtype=h_dt)
    wr = rnd(e, width, dtype=w_dt, seed=1, scale=0.2)
    wr[7] = wr[2]                      # experts 2 and 7 always tie: the lower id must win
    wg = rnd(1, width, dtype=w_dt, seed=2, scale=0.2)
    ids = torch.empty(n, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, k, device=DEV)
    gate = torch.empty(n, device=DEV)
    probs = torch.empty(n, e, device=DEV)
    st = status()
    ops.router_topk(h, wr, wg, ids, wts, gate, k, norm, st, probs)
    assert st.item() == 0
    p = torch.softmax(h.double() @ wr.double().t(), -1)
    close(probs, p, torch.float32, "probabilities")
    close(gate, torch.sigmoid(h.double() @ wg.double().t())[:, 0], torch.float32, "shared gate")
    order = np.argsort(-p.cpu().numpy(), axis=1, kind="stable")[:, :k]
    got = ids.cpu().numpy()
    for t in range(n):
        assert list(got[t]) == list(order[t]), (t, got[t], order[t])
        assert not (7 in got[t] and 2 not in got[t])
        chosen = p[t, got[t]]
        close(wts[t], chosen / chosen.sum() if norm else chosen, torch.float32, "weights")


@pytest.mark.parametrize("w_dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, e, k, norm", [(1, 10, 3, False), (8, 60, 4, False), (32, 7, 7, True), (13, 64, 8, True),
                                           (64, 60, 4, False), (50, 12, 3, True)])
def test_route_small_equals_router_and_permutation(w_dt, n, e, k, norm):
    """The two-launch path for few tokens gives what router_topk + moe_permute give."""
    width = 200
    h = rnd(n, width)
    wr = rnd(e, width, dtype=w_dt, seed=1, scale=0.3)
    if e > 7:
        wr[7] = wr[2]
    wg = rnd(1, width, dtype=w_dt, seed=2, scale=0.3)
    i32 = lambda *shape: torch.empty(*shape, dtype=torch.int32, device=DEV)
    f32 = lambda *shape: torch.empty(*shape, device=DEV)
    ids_a, w_a, gate_a, probs_a, st = i32(n, k), f32(n, k), f32(n), f32(n, e), status()
    ops.router_topk(h, wr, wg, ids_a, w_a, gate_a, k, norm, st, probs_a)
    ids_b, w_b, gate_b, probs_b = i32(n, k), f32(n, k), f32(n), f32(n, e)
    offsets, perm_token, perm_weight, inverse = i32(e + 1), i32(n * k), f32(n * k), i32(n, k)
    ops.route_small(h, wr, wg, f32(n, e + 1), ids_b, w_b, gate_b, k, norm, offsets, perm_token, perm_weight, inverse, st,
                    probs_b)
    assert st.item() == 0
    assert torch.equal(ids_a, ids_b)
    close(w_b, w_a, torch.float32, "routing weights")
    close(gate_b, gate_a, torch.float32, "shared gate")
    close(probs_b, probs_a, torch.float32, "probabilities")
    ids_np, off = ids_b.cpu().numpy(), offsets.cpu().numpy()
    assert list(off) == list(np.concatenate([[0], np.cumsum(np.bincount(ids_np.reshape(-1), minlength=e))]))
    # with the tile list of the grouped tensor-core products: what moe_permute lists for the same choices
    tiles_a = (i32(n * k + e), i32(n * k + e), i32(n * k + e), i32(1))
    tiles_b = (i32(n * k + e), i32(n * k + e), i32(n * k + e), i32(1))
    ops.moe_permute(ids_b, w_b, e, i32(e + 1), i32(n * k), f32(n * k), i32(n, k), st, tiles=tiles_a)
    ops.route_small(h, wr, wg, f32(n, e + 1), i32(n, k), f32(n, k), f32(n), k, norm, i32(e + 1), i32(n * k), f32(n * k),
                    i32(n, k), st, tiles=tiles_b)
    n_t = int(tiles_a[3].item())
    assert st.item() == 0 and int(tiles_b[3].item()) == n_t == int((np.bincount(ids_np.reshape(-1), minlength=e) > 0).sum())
    for x, y in zip(tiles_a[:3], tiles_b[:3]):
        assert torch.equal(x[:n_t], y[:n_t])
    inv, pt, pw = inverse.cpu().numpy(), perm_token.cpu().numpy(), perm_weight.cpu().numpy()
    assert sorted(inv.reshape(-1)) == list(range(n * k))
    for t in range(n):
        for r in range(k):
            row = inv[t, r]
            assert off[ids_np[t, r]] <= row < off[ids_np[t, r] + 1] and pt[row] == t and pw[row] == w_b[t, r].item()


def test_moe_permute_and_combine():
    n, k, e, width = 37, 3, 6, 50
    rng = np.random.default_rng(0)
    ids_np = np.stack([rng.permutation(e)[:k] for _ in range(n)]).astype(np.int32)
    ids_np[:, :] = np.where(ids_np == 4, 5, ids_np) if False else ids_np
    ids = torch.tensor(ids_np, device=DEV)
    wts = rnd(n, k).abs()
    offsets = torch.empty(e + 1, dtype=torch.int32, device=DEV)
    perm_token = torch.empty(n * k, dtype=torch.int32, device=DEV)
    perm_weight = torch.empty(n * k, device=DEV)
    inverse = torch.empty(n, k, dtype=torch.int32, device=DEV)
    st = status()
    ops.moe_permute(ids, wts, e, offsets, perm_token, perm_weight, inverse, st)
    assert st.item() == 0
    off = offsets.cpu().numpy()
    assert list(off) == list(np.concatenate([[0], np.cumsum(np.bincount(ids_np.reshape(-1), minlength=e))]))
    inv, pt, pw = inverse.cpu().numpy(), perm_token.cpu().numpy(), perm_weight.cpu().numpy()
    assert sorted(inv.reshape(-1)) == list(range(n * k)), "a permuted row is used twice or not at all"
    for t in range(n):
        for r in range(k):
            row = inv[t, r]
            assert off[ids_np[t, r]] <= row < off[ids_np[t, r] + 1] and pt[row] == t
            assert pw[row] == wts[t, r].item()
    expert_out = rnd(n * k, width, seed=3)
    shared, gate = rnd(n, width, seed=4), rnd(n, seed=5).abs()
    y = torch.empty(n, width, device=DEV)
    ops.moe_combine(expert_out, ids, inverse, gate, shared, y)
    eo = expert_out.cpu().numpy()
    for t in range(n):
        acc = np.zeros(width, dtype=np.float32)
        for r in np.argsort(ids_np[t], kind="stable"):          # ascending expert id, float32 adds in that order
            acc = acc + eo[inv[t, r]]
        acc = acc + gate[t].item() * shared[t].cpu().numpy()
        assert np.allclose(y[t].cpu().numpy(), acc, rtol=0, atol=1e-6), t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [200, 2048])
def test_combine_add_norm_in_one_kernel_gives_the_same_bits(dtype, width):
    n, k, e = 19, 3, 6
    rng = np.random.default_rng(1)
    ids = torch.tensor(np.stack([rng.permutation(e)[:k] for _ in range(n)]).astype(np.int32), device=DEV)
    inverse = torch.tensor(rng.permutation(n * k).reshape(n, k).astype(np.int32), device=DEV)
    expert_out, shared, gate = rnd(n * k, width, seed=3), rnd(n, width, seed=4), rnd(n, seed=5).abs()
    x, gamma = rnd(n, width, seed=6), 1 + 0.1 * rnd(width, seed=7)
    y = torch.empty(n, width, device=DEV)
    ops.moe_combine(expert_out, ids, inverse, gate, shared, y)
    x_ref, h_ref, h32_ref = x.clone(), torch.empty(n, width, dtype=dtype, device=DEV), torch.empty(n, width, device=DEV)
    ops.add_rmsnorm(x_ref, y, gamma, h_ref, 1e-6, h32=h32_ref)
    x_got, h_got, h32_got = x.clone(), torch.empty_like(h_ref), torch.empty_like(h32_ref)
    ops.moe_combine_add_rmsnorm(expert_out, ids, inverse, gate, shared, x_got, gamma, h_got, 1e-6, h32=h32_got)
    assert torch.equal(x_got, x_ref) and torch.equal(h_got, h_ref) and torch.equal(h32_got, h32_ref)
    rows = torch.tensor([4, 0, 18], dtype=torch.int32, device=DEV)
    h_ref2, h_got2, x_keep = torch.empty(3, width, dtype=dtype, device=DEV), torch.empty(3, width, dtype=dtype, device=DEV), x.clone()
    ops.add_rmsnorm(x.clone(), y, gamma, h_ref2, 1e-6, rows=rows, write_x=False)
    ops.moe_combine_add_rmsnorm(expert_out, ids, inverse, gate, shared, x_keep, gamma, h_got2, 1e-6, rows=rows, write_x=False)
    assert torch.equal(h_got2, h_ref2) and torch.equal(x_keep, x)


def test_argmax_takes_the_lower_id_on_ties():
    logits = rnd(4, 1000)
    logits[0, 900] = logits[0, 17] = 50.0
    logits[1, 999] = 60.0
    logits[2, 0] = 60.0
    tokens = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.pick_tokens(logits, None, None, torch.zeros(4, dtype=torch.int64, device=DEV),
                    torch.arange(4, dtype=torch.int32, device=DEV), tokens)
    assert tokens.tolist() == [17, 999, 0, int(logits[3].argmax())]


def _draw_setup(rows, vocab):
    logits = rnd(rows, vocab, scale=2.0)
    temps = [0.8 if r % 3 else 1.5 for r in range(rows)]
    temps[5] = 0.0
    top_ps = [None if r % 2 else [0.9, 0.5, 0.05][r % 3] for r in range(rows)]
    seeds = [1000 + 7 * r for r in range(rows)]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    tokens = torch.empty(rows, dtype=torch.int32, device=DEV)
    args = (logits, torch.tensor(temps, device=DEV), torch.tensor([-1.0 if t is None else t for t in top_ps], device=DEV),
            state, torch.arange(rows, dtype=torch.int32, device=DEV), tokens)
    return logits, temps, top_ps, seeds, state, tokens, args


def test_sampling_matches_the_plain_sampler():
    """Same seed, same logits: the device picks what the plain sampler picks,
    with and without a nucleus cut, and advances its stream by one draw."""
    rows, vocab = 48, 1000
    logits, temps, top_ps, seeds, state, tokens, args = _draw_setup(rows, vocab)
    ops.pick_tokens(*args)
    first = tokens.tolist()
    ops.pick_tokens(*args)
    second = tokens.tolist()
    lg = logits.cpu().numpy()
    for r in range(rows):
        rng = plain.SplitMix64(seeds[r])
        if temps[r] == 0.0:
            assert first[r] == second[r] == int(lg[r].argmax())
            assert state[r].item() == seeds[r], "a greedy row must not draw"
            continue
        assert first[r] == plain.sample_row(lg[r], temps[r], top_ps[r], rng), f"row {r}, first draw"
        assert second[r] == plain.sample_row(lg[r], temps[r], top_ps[r], rng), f"row {r}, second draw"
        assert (state[r].item() & ((1 << 64) - 1)) == rng.state


def test_sampling_at_a_large_flat_vocabulary_picks_the_token_under_the_draw():
    """With 151,936 nearly equal weights the plain sampler's running float32
    sums drift by more than one token's mass, so equality with it is not a
    property of a correct sampler.  What is: the chosen token's interval of
    cumulative mass (ranking by descending weight, ties by id; sums in
    float64) holds the draw u * (kept mass), up to the rounding of u."""
    rows, vocab = 24, 151936
    logits, temps, top_ps, seeds, state, tokens, args = _draw_setup(rows, vocab)
    ops.pick_tokens(*args)
    picked = tokens.tolist()
    lg = logits.cpu().numpy()
    for r in range(rows):
        if temps[r] == 0.0:
            assert picked[r] == int(lg[r].argmax())
            continue
        u = np.float32(plain.SplitMix64(seeds[r]).next_f64())
        w = np.exp((lg[r] - lg[r].max()) * (np.float32(1.0) / np.float32(temps[r]))).astype(np.float32)
        order = np.lexsort((np.arange(vocab), -w))
        cum = np.cumsum(w[order].astype(np.float64))
        kept = cum[-1]
        if top_ps[r] is not None:
            keep = int(np.argmax(cum >= kept * top_ps[r]))
            kept = cum[keep]
            assert np.nonzero(order == picked[r])[0][0] <= keep, f"row {r}: picked outside the nucleus"
        rank = int(np.nonzero(order == picked[r])[0][0])
        thr, tol = float(u) * kept, 1e-6 * kept
        assert cum[rank] >= thr - tol and (rank == 0 or cum[rank - 1] <= thr + tol), (
            f"row {r}: draw {thr:.6f} is outside [{cum[rank - 1] if rank else 0:.6f}, {cum[rank]:.6f}]")


def test_sampling_follows_the_distribution():
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]], device=DEV).repeat(4096, 1).contiguous()
    state = torch.arange(4096, dtype=torch.int64, device=DEV) * 7919 + 3
    tokens = torch.empty(4096, dtype=torch.int32, device=DEV)
    ops.pick_tokens(logits, torch.ones(4096, device=DEV), None, state, torch.arange(4096, dtype=torch.int32, device=DEV),
                    tokens)
    freq = np.bincount(tokens.cpu().numpy(), minlength=5) / 4096
    p = torch.softmax(logits[0].double(), 0).cpu().numpy()
    assert np.abs(freq - p).max() < 0.03


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_normal_fill_matches_the_host_generator(dtype):
    out = torch.empty(5000, dtype=dtype, device=DEV)
    ops.normal_fill(out, 0x1234567890ABCDEF, 1.0, 0.5)
    host = torch.from_numpy(normal_values(0x1234567890ABCDEF, 5000, 1.0, 0.5)).to(dtype)
    diff = (out.cpu().float() - host.float()).abs()
    assert diff.max() <= (1e-5 if dtype == torch.float32 else 2.0 ** -7 * 3)
    assert abs(out.float().mean().item() - 1.0) < 0.03 and abs(out.float().std().item() - 0.5) < 0.03


def test_finite_check_sets_the_status_word():
    st = status()
    v = rnd(3, 1000)
    ops.finite_check(v, st)
    assert st.item() == 0
    v[1, 500] = float("nan")
    ops.finite_check(v, st)
    assert st.item() == 2


# ---------------------------------------------------------------------------
# bfloat16 kernels
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 5, 8, 13, 16, 40])
@pytest.mark.parametrize("n, k", [(70, 96), (130, 200), (48, 2048), (33, 5632)])
def test_gemm_skinny_dense(m, n, k):
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1)
    scale = rnd(m, seed=2)
    c = torch.full((m + 2, n), 7.0, device=DEV)
    ops.gemm_skinny(a, w, c, row_scale=scale, rows=m)
    close(c[:m], (a.double() @ w.double().t()) * scale.double()[:, None], torch.float32, "skinny dense", k=k)
    assert torch.all(c[m:] == 7.0)
    # a row's bits do not depend on the rows beside it
    c1 = torch.empty(1, n, device=DEV)
    ops.gemm_skinny(a[m - 1:m], w, c1, row_scale=scale[m - 1:m].contiguous())
    assert torch.equal(c1[0], c[m - 1])


@pytest.mark.parametrize("n", [8000, 16000])
def test_gemm_skinny_two_and_four_warps_per_tile(n):
    """Between few tiles (eight warps share one) and many (one each): 500 tiles -> four, 1000 -> two."""
    m, k = 7, 200
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1)
    c = torch.empty(m, n, device=DEV)
    ops.gemm_skinny(a, w, c)
    close(c, a.double() @ w.double().t(), torch.float32, f"{n} rows of weights", k=k)
    inter = n // 2
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(a, w, act, swiglu=True)
    g, u = a.double() @ w[:inter].double().t(), a.double() @ w[inter:].double().t()
    close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16, "swiglu")


def test_gemm_skinny_many_tiles_one_tile_per_warp():
    """With enough tiles of weight rows each warp takes a tile of its own and walks all of K: dense,
    fused SwiGLU and grouped with a ragged last tile."""
    m, n, k = 5, 120001, 72
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1)
    scale = rnd(m, seed=2)
    c = torch.empty(m, n, device=DEV)
    ops.gemm_skinny(a, w, c, row_scale=scale)
    close(c, (a.double() @ w.double().t()) * scale.double()[:, None], torch.float32, "one tile per warp, dense", k=k)
    inter = 60000
    w2 = rnd(2 * inter, k, dtype=torch.bfloat16, seed=3, scale=0.3)
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(a, w2, act, swiglu=True)
    g, u = a.double() @ w2[:inter].double().t(), a.double() @ w2[inter:].double().t()
    close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16, "one tile per warp, swiglu")
    groups, n3 = 40, 2900
    counts = [(3 * i) % 5 for i in range(groups)]
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    total = sum(counts)
    a3 = rnd(total, k, dtype=torch.bfloat16, seed=4)
    w3 = rnd(groups, n3, k, dtype=torch.bfloat16, seed=5)
    c3 = torch.empty(total, n3, device=DEV)
    ops.gemm_skinny(a3, w3, c3, group_offsets=offsets, rows=total, max_rows=4)
    row = 0
    for e, cnt in enumerate(counts):
        if cnt:
            close(c3[row:row + cnt], a3[row:row + cnt].double() @ w3[e].double().t(), torch.float32, f"group {e}", k=k)
        row += cnt


@pytest.mark.parametrize("m, inter, k", [(3, 44, 96), (16, 100, 2048), (9, 8, 64)])
def test_gemm_skinny_swiglu(m, inter, k):
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.2)
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(a, w, act, swiglu=True)
    g, u = a.double() @ w[:inter].double().t(), a.double() @ w[inter:].double().t()
    close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16, "skinny swiglu")


def test_gemm_skinny_grouped_gather_scale_and_chunks():
    g, n, k = 6, 40, 136
    counts = [2, 0, 37, 1, 0, 9]                      # 37 rows: more than one staging chunk
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    total = sum(counts)
    src = rnd(20, k, dtype=torch.bfloat16)
    a_rows = torch.tensor(np.random.default_rng(1).integers(0, 20, total), dtype=torch.int32, device=DEV)
    w = rnd(g, n, k, dtype=torch.bfloat16, seed=1)
    scale = rnd(total, seed=2)
    c = torch.full((total + 1, n), 7.0, device=DEV)
    ops.gemm_skinny(src, w, c, a_rows=a_rows, row_scale=scale, group_offsets=offsets, rows=total, max_rows=20)
    row = 0
    for e, cnt in enumerate(counts):
        for _ in range(cnt):
            ref = (src[a_rows[row].long()].double() @ w[e].double().t()) * scale[row].double()
            close(c[row], ref, torch.float32, f"group {e} row {row}")
            row += 1
    assert torch.all(c[total:] == 7.0)
    # grouped swiglu, rows in place (no gather)
    inter = 24
    w2 = rnd(g, 2 * inter, k, dtype=torch.bfloat16, seed=3, scale=0.3)
    a2 = rnd(total, k, dtype=torch.bfloat16, seed=4)
    act = torch.empty(total, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(a2, w2, act, swiglu=True, group_offsets=offsets, rows=total, max_rows=37)
    row = 0
    for e, cnt in enumerate(counts):
        for _ in range(cnt):
            gg, uu = a2[row].double() @ w2[e, :inter].double().t(), a2[row].double() @ w2[e, inter:].double().t()
            close(act[row], gg / (1 + torch.exp(-gg)) * uu, torch.bfloat16, f"swiglu group {e} row {row}")
            row += 1


@pytest.mark.parametrize("counts_at", [{0: 1, 17: 2, 59: 1}, {59: 4}, {3: 1, 4: 1, 5: 1, 58: 1}, {0: 5}])
def test_gemm_skinny_grouped_fewer_rows_than_groups(counts_at):
    """A decode step of one sequence names a few experts of many: the grid then has one row per (token,
    expert) pair and finds each pair's group; the first and the last group, neighbours, one group with
    every row."""
    g, n, k, inter = 60, 50, 136, 24
    counts = [counts_at.get(e, 0) for e in range(g)]
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    total = sum(counts)
    assert total < g
    src = rnd(7, k, dtype=torch.bfloat16)
    a_rows = torch.tensor(np.random.default_rng(2).integers(0, 7, total), dtype=torch.int32, device=DEV)
    w = rnd(g, n, k, dtype=torch.bfloat16, seed=1)
    scale = rnd(total, seed=2)
    c = torch.full((total + 1, n), 7.0, device=DEV)
    ops.gemm_skinny(src, w, c, a_rows=a_rows, row_scale=scale, group_offsets=offsets, rows=total, max_rows=8)
    w2 = rnd(g, 2 * inter, k, dtype=torch.bfloat16, seed=3, scale=0.3)
    act = torch.full((total + 1, inter), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(src, w2, act, swiglu=True, a_rows=a_rows, group_offsets=offsets, rows=total, max_rows=8)
    row = 0
    for e, cnt in enumerate(counts):
        for _ in range(cnt):
            x = src[a_rows[row].long()].double()
            close(c[row], (x @ w[e].double().t()) * scale[row].double(), torch.float32, f"group {e} row {row}")
            gg, uu = x @ w2[e, :inter].double().t(), x @ w2[e, inter:].double().t()
            close(act[row], gg / (1 + torch.exp(-gg)) * uu, torch.bfloat16, f"swiglu group {e} row {row}")
            row += 1
    assert torch.all(c[total:] == 7.0) and torch.all(act[total:] == 7.0)


@pytest.mark.parametrize("split", [128, 256, 512, 1024])
@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 4, 128, None), (6, 2, 64, None), (7, 1, 128, 100), (8, 1, 192, None),
                                                 (4, 2, 256, 300), (16, 16, 128, 65)])
def test_attn_decode_finds_the_key_that_matters(nh, nkv, hd, window, split):
    """The split-key kernel on the same kind of made-up cache as the plain one:
    far keys, keys at the window's edges, at page and split boundaries, other
    sequences in interleaved pages."""
    torch.manual_seed(2)
    dtype = torch.bfloat16
    lens = [700, 300, 65]
    group = nh // nkv
    tables = [[3 * i + s for i in range(12)] for s in range(3)]
    ks = [torch.randn(n, nkv, hd) * 0.3 for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    queries = []
    last = lens[0] - 1
    w = window or 10 ** 9
    for target in {3, 63, 64, 255, 256, 257, 511, 512, max(0, last - w + 1), max(0, last - w), last}:
        queries.append((0, last, target))
    queries += [(1, 299, 256), (1, 256, 255), (1, 255, 0), (2, 64, 63), (2, 0, 0), (2, 1, 0)]
    q = torch.randn(len(queries), nh, hd) * 0.3
    for i, (s, p, target) in enumerate(queries):
        for h in range(nh):
            ks[s][target, h // group] = ks[s][target, h // group] / ks[s][target, h // group].norm() * 6.0
            q[i, h] = ks[s][target, h // group] * (np.sqrt(hd) * 3.0 / 6.0)
    qd = q.to(dtype)
    kc, vc = paged(ks, vs, tables, 36, nkv, hd, dtype)
    table = torch.tensor(tables, dtype=torch.int32, device=DEV)
    n = len(queries)
    out = torch.empty(n, nh * hd, dtype=dtype, device=DEV)
    n_splits = (700 + split - 1) // split
    part_o = torch.full((n, nh, n_splits, hd), float("nan"), device=DEV)
    part_ml = torch.full((n, nh, n_splits, 2), float("nan"), device=DEV)
    st = status()
    counters = torch.zeros(n * nh, dtype=torch.int32, device=DEV)
    ops.attn_decode(qd.reshape(n, nh * hd).to(DEV), kc, vc, out, part_o, part_ml, counters,
                    torch.tensor([s for s, _, _ in queries], dtype=torch.int32, device=DEV),
                    torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=DEV), table, 64, nh, nkv, hd,
                    window, split, n_splits, st)
    assert st.item() == 0 and not counters.any(), "the counters must be left at zero"
    for i, (s, p, target) in enumerate(queries):
        ref = attention_reference(qd[i].float(), ks[s].to(dtype).float(), vs[s].to(dtype).float(), p, window, group)
        close(out[i].view(nh, hd), ref, dtype, f"query {i} (sequence {s}, position {p}, target key {target})")


@pytest.mark.parametrize("split", [192, 640, 1024])
@pytest.mark.parametrize("nh, nkv, hd, window", [(7, 1, 128, None), (4, 4, 128, 1500), (6, 2, 64, None), (2, 1, 256, 1030)])
def test_attn_decode_over_many_splits_of_a_long_sequence(nh, nkv, hd, window, split):
    """2,500 positions in scattered pages: keys that matter at the boundaries of the 1,024-position splits, at the
    window's edge and at both ends; the combine of the row's splits (up to ten here, seven heads to a block in the
    first case) against the float64 reference."""
    torch.manual_seed(5)
    dtype = torch.bfloat16
    length, group = 2500, nh // nkv
    pages = (length + 63) // 64
    order = torch.randperm(pages + 3).tolist()
    tables = [order[:pages]]
    ks, vs = [torch.randn(length, nkv, hd) * 0.3], [torch.randn(length, nkv, hd)]
    last = length - 1
    w = window or 10 ** 9
    targets = sorted({0, 1023, 1024, 1025, 2047, 2048, 2304, max(0, last - w + 1), max(0, last - w), last})
    queries = [(0, last, t) for t in targets] + [(0, 1024, 1023), (0, 1024, 1024), (0, 1023, 0), (0, 2048, 1024)]
    q = torch.randn(len(queries), nh, hd) * 0.3
    for i, (s, p, target) in enumerate(queries):
        for h in range(nh):
            ks[s][target, h // group] = ks[s][target, h // group] / ks[s][target, h // group].norm() * 6.0
            q[i, h] = ks[s][target, h // group] * (np.sqrt(hd) * 3.0 / 6.0)
    qd = q.to(dtype)
    kc, vc = paged(ks, vs, tables, pages + 3, nkv, hd, dtype)
    table = torch.tensor(tables, dtype=torch.int32, device=DEV)
    n = len(queries)
    out = torch.empty(n, nh * hd, dtype=dtype, device=DEV)
    n_splits = (length + split - 1) // split
    part_o = torch.full((n, nh, n_splits, hd), float("nan"), device=DEV)
    part_ml = torch.full((n, nh, n_splits, 2), float("nan"), device=DEV)
    st = status()
    counters = torch.zeros(n * nh, dtype=torch.int32, device=DEV)
    ops.attn_decode(qd.reshape(n, nh * hd).to(DEV), kc, vc, out, part_o, part_ml, counters,
                    torch.zeros(n, dtype=torch.int32, device=DEV),
                    torch.tensor([p for _, p, _ in queries], dtype=torch.int32, device=DEV), table, 64, nh, nkv, hd,
                    window, split, n_splits, st)
    assert st.item() == 0 and not counters.any(), "the counters must be left at zero"
    for i, (s, p, target) in enumerate(queries):
        ref = attention_reference(qd[i].float(), ks[s].to(dtype).float(), vs[s].to(dtype).float(), p, window, group)
        close(out[i].view(nh, hd), ref, dtype, f"query {i} (position {p}, target key {target})")


@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 4, 128, None), (6, 2, 64, None), (4, 1, 24, 16), (2, 1, 128, 100),
                                                 (4, 2, 16, None), (3, 1, 80, 65)])
def test_attn_prefill_against_reference(nh, nkv, hd, window):
    """Runs of new tokens of unequal length, some continuing a cached past, in
    interleaved pages; in every sequence some keys are made to dominate so that
    a lost, shifted or wrongly masked key shows."""
    check_attn_prefill(ops.attn_prefill, nh, nkv, hd, window)


@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 4, 128, None), (6, 2, 64, None), (2, 1, 128, 100), (3, 1, 64, 65),
                                                 (2, 2, 128, 300)])
def test_attn_prefill_tc05_against_reference(nh, nkv, hd, window):
    """The same runs through the kernel that keeps scores and weighted values in tensor memory."""
    check_attn_prefill(ops.attn_prefill_tc05, nh, nkv, hd, window, tile=ops.ATTN_TC05_TILE_ROWS)


def check_attn_prefill(fn, nh, nkv, hd, window, tile=64, runs=None):
    torch.manual_seed(3)
    dtype = torch.bfloat16
    group = nh // nkv
    runs = runs or [(0, 200), (130, 70), (0, 1), (63, 66), (300, 129), (10, 420)]        # (past, new)
    lens = [p + n for p, n in runs]
    n_seq, per_seq = len(runs), (max(lens) + 63) // 64
    tables = [[n_seq * i + s for i in range(per_seq)] for s in range(n_seq)]
    ks = [torch.randn(n, nkv, hd) * 0.3 for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    qs = [torch.randn(n, nh, hd) * 0.3 for _p, n in runs]
    rng = np.random.default_rng(0)
    for s, (past, new) in enumerate(runs):
        for _ in range(12):                                            # a dozen (query, key) pairs that stand out
            i = int(rng.integers(0, new))
            pos = past + i
            lo = 0 if not window else max(0, pos - window + 1)
            target = int(rng.choice([lo, pos, (lo + pos) // 2, max(lo, pos - 63), max(lo, pos - 64), max(lo, (pos // 64) * 64)]))
            for h in range(nh):
                ks[s][target, h // group] = ks[s][target, h // group] / ks[s][target, h // group].norm() * 6.0
                qs[s][i, h] = ks[s][target, h // group] * (np.sqrt(hd) * 3.0 / 6.0)
    kc, vc = paged(ks, vs, tables, n_seq * per_seq, nkv, hd, dtype)
    q = torch.cat(qs).to(dtype)
    n = q.shape[0]
    out = torch.full((n, nh * hd), float("nan"), dtype=dtype, device=DEV)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    starts = np.concatenate([[0], np.cumsum([nw for _p, nw in runs])])
    st = status()
    fn(q.reshape(n, nh * hd).to(DEV), kc, vc, out,
       i32([s for s, (_p, nw) in enumerate(runs) for _ in range(0, nw, tile)]),
       i32([f for _p, nw in runs for f in range(0, nw, tile)]), i32(starts), i32([p for p, _n in runs]),
       i32(tables), 64, nh, nkv, hd, window, st)
    assert st.item() == 0
    for s, (past, new) in enumerate(runs):
        for i in range(new):
            ref = attention_reference(q[starts[s] + i].float(), ks[s].to(dtype).float(), vs[s].to(dtype).float(),
                                      past + i, window, group)
            close(out[starts[s] + i].view(nh, hd), ref, dtype, f"sequence {s}, new token {i} (position {past + i})")


# ---------------------------------------------------------------------------
# TMA + tcgen05 products
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("m, n, k", [(128, 128, 64), (256, 128, 256), (300, 200, 2048), (77, 130, 200), (1, 24, 8),
                                     (513, 384, 1408), (17, 129, 72)])
def test_gemm_tc05_dense(m, n, k):
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, seed=1)
    scale = rnd(m, seed=2)
    c = torch.full((m + 3, n), 7.0, device=DEV)
    st = status()
    ops.gemm_tc05(a, w, c, st, row_scale=scale, rows=m)
    assert st.item() == 0
    close(c[:m], (a.double() @ w.double().t()) * scale.double()[:, None], torch.float32, "tcgen05 dense", k=k)
    assert torch.all(c[m:] == 7.0), "rows beyond the product were written"


@pytest.mark.parametrize("m, inter, k", [(128, 64, 64), (200, 100, 192), (64, 1408, 2048)])
def test_gemm_tc05_swiglu(m, inter, k):
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    st = status()
    ops.gemm_tc05(a, w, act, st, swiglu=True)
    assert st.item() == 0
    g, u = a.double() @ w[:inter].double().t(), a.double() @ w[inter:].double().t()
    close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16, "tcgen05 swiglu")


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("max_ctas", [2, 7, 140])
def test_gemm_tc05_on_fewer_ctas_than_sms_gives_the_same_bits(pair, max_ctas):
    """A launch told to take at most ``max_ctas`` SMs (so that another stream's kernels find room) walks the
    same tiles with a longer stride: equal bits, for an odd k-step count too (groups of two k steps then
    straddle tiles)."""
    m, inter, k = 700, 328, 3 * 64 + 8          # 4 k steps, the last one 8 wide
    a, w = rnd(m, k, dtype=torch.bfloat16), rnd(2 * inter, k, dtype=torch.bfloat16, seed=1, scale=0.1)
    outs = []
    for limit in (0, max_ctas):
        act = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
        c = torch.zeros(m, 2 * inter, device=DEV)
        st = status()
        ops.gemm_tc05(a, w, act, st, swiglu=True, pair=pair, max_ctas=limit)
        ops.gemm_tc05(a, w, c, st, pair=pair, max_ctas=limit)
        assert st.item() == 0
        outs.append((act, c))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    close(outs[1][1], a.double() @ w.double().t(), torch.float32, "tcgen05 dense on few CTAs", k=k)
    with pytest.raises(Exception):
        ops.gemm_tc05(a, w, outs[0][1], status(), pair=True, max_ctas=1)      # a pair needs two


def check_tile_cover(first_rows, counts, rows, tile):
    """Every permuted row lies in exactly one tile."""
    seen = np.zeros(rows, dtype=np.int64)
    for r, c in zip(first_rows, counts):
        seen[r:r + c] += 1
    assert np.all(seen == 1), "a row outside every tile or in two"


def test_gemm_tc05_grouped_through_the_permutation():
    """Router output -> permutation and tile list -> gathered rows -> grouped SwiGLU product -> grouped
    down product with the routing weight; experts with no rows, one row and several tiles of rows."""
    n_tok, k_top, e, width, inter = 700, 2, 7, 136, 72
    rng = np.random.default_rng(0)
    probs = np.array([0.55, 0.0, 0.25, 0.001, 0.1, 0.0, 0.099])
    ids_np = np.stack([rng.choice(e, size=k_top, replace=False, p=probs) for _ in range(n_tok)]).astype(np.int32)
    ids = torch.tensor(ids_np, device=DEV)
    wts = rnd(n_tok, k_top).abs() + 0.1
    rows = n_tok * k_top
    i32 = lambda *shape: torch.empty(*shape, dtype=torch.int32, device=DEV)
    offsets, perm_token, inverse = i32(e + 1), i32(rows), i32(n_tok, k_top)
    perm_weight = torch.empty(rows, device=DEV)
    tile = ops.TC05_TILE_ROWS
    max_tiles = (rows + tile - 1) // tile + e
    tiles = (i32(max_tiles), i32(max_tiles), i32(max_tiles), i32(1))
    st = status()
    ops.moe_permute(ids, wts, e, offsets, perm_token, perm_weight, inverse, st, tiles=tiles)
    off = offsets.cpu().numpy()
    n_tiles = tiles[3].item()
    assert n_tiles == sum((off[i + 1] - off[i] + tile - 1) // tile for i in range(e))
    tg, tr, tc = (t.cpu().numpy()[:n_tiles] for t in tiles[:3])
    assert all(off[g] <= r and r + c <= off[g + 1] and 0 < c <= tile for g, r, c in zip(tg, tr, tc))
    check_tile_cover(tr, tc, rows, tile)
    h = rnd(n_tok, width, dtype=torch.bfloat16, seed=5)
    h_perm = torch.empty(rows, width, dtype=torch.bfloat16, device=DEV)
    ops.gather_rows(h, perm_token, h_perm)
    assert torch.equal(h_perm, h[perm_token.long()])
    w_gu = rnd(e, 2 * inter, width, dtype=torch.bfloat16, seed=6, scale=0.2)
    w_d = rnd(e, width, inter, dtype=torch.bfloat16, seed=7, scale=0.2)
    act = torch.empty(rows, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc05(h_perm, w_gu, act, st, swiglu=True, tiles=tiles)
    out = torch.empty(rows, width, device=DEV)
    ops.gemm_tc05(act, w_d, out, st, row_scale=perm_weight, tiles=tiles)
    assert st.item() == 0
    for g in range(e):
        lo, hi = off[g], off[g + 1]
        if lo == hi:
            continue
        x = h_perm[lo:hi].double()
        gg, uu = x @ w_gu[g, :inter].double().t(), x @ w_gu[g, inter:].double().t()
        close(act[lo:hi], gg / (1 + torch.exp(-gg)) * uu, torch.bfloat16, f"expert {g} gate/up")
        ref = (act[lo:hi].double() @ w_d[g].double().t()) * perm_weight[lo:hi].double()[:, None]
        close(out[lo:hi], ref, torch.float32, f"expert {g} down", k=inter)


@pytest.mark.parametrize("tile_rows", [128, 256])
@pytest.mark.parametrize("counts", [
    [80] * 9,                                   # stages of 26 KB: eight of them end exactly at the ring's end
    [137, 9, 256, 1, 300, 16, 200, 33, 77, 128, 145, 250],
    [16, 240, 48, 176, 112, 96, 208, 64],       # every width of stage in turn
])
def test_gemm_tc05_grouped_stages_of_many_widths(tile_rows, counts):
    """The ring of stages is a byte queue whose stages are as wide as their tile: tiles of many widths in a
    row, long enough in k that the ring turns over many times, against the dense product of each group."""
    e, width, inter = len(counts), 64 * 13, 64 * 3 + 40
    mk = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    g, r0, rc, off = [], [], [], [0]
    for grp, c in enumerate(counts):
        for s0 in range(0, c, tile_rows):
            g.append(grp), r0.append(off[-1] + s0), rc.append(min(tile_rows, c - s0))
        off.append(off[-1] + c)
    rows = off[-1]
    tiles = (mk(g), mk(r0), mk(rc), mk([len(g)]))
    x = rnd(rows, width, dtype=torch.bfloat16, seed=3)
    w_gu = rnd(e, 2 * inter, width, dtype=torch.bfloat16, seed=6, scale=0.1)
    w_d = rnd(e, width, inter, dtype=torch.bfloat16, seed=7, scale=0.2)
    scale = rnd(rows, seed=8).abs() + 0.1
    st = status()
    act = torch.full((rows + 2, inter), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc05(x, w_gu, act, st, swiglu=True, tiles=tiles, rows=rows, tile_rows=tile_rows)
    out = torch.full((rows + 2, width), 5.0, device=DEV)
    ops.gemm_tc05(act, w_d, out, st, row_scale=scale, tiles=tiles, rows=rows, tile_rows=tile_rows)
    assert st.item() == 0
    assert torch.all(act[rows:] == 3.0) and torch.all(out[rows:] == 5.0), "rows beyond the product were written"
    for grp in range(e):
        lo, hi = off[grp], off[grp + 1]
        xx = x[lo:hi].double()
        gg, uu = xx @ w_gu[grp, :inter].double().t(), xx @ w_gu[grp, inter:].double().t()
        close(act[lo:hi], gg / (1 + torch.exp(-gg)) * uu, torch.bfloat16, f"group {grp} gate/up")
        ref = (act[lo:hi].double() @ w_d[grp].double().t()) * scale[lo:hi].double()[:, None]
        close(out[lo:hi], ref, torch.float32, f"group {grp} down", k=inter)


@pytest.mark.parametrize("n, width, e, k, with_gate", [(700, 256, 60, 4, True), (65, 128, 64, 8, True), (300, 384, 7, 2, False),
                                                        (2048, 2048, 60, 4, True)])
def test_router_on_tensor_cores_keeps_32_bit_precision(n, width, e, k, with_gate):
    """Many tokens, 32-bit activations, bfloat16 weights: the logits come from mma.sync over three bfloat16 parts of
    every activation.  They must be as good as a 32-bit dot product (far better than bfloat16 activations would
    give), ties must still go to the lower id, and the choices must be those of the exact probabilities."""
    h = rnd(n, width) * 3.0
    wr = rnd(e, width, dtype=torch.bfloat16, seed=1, scale=0.2)
    if e > 5:
        wr[5] = wr[2]                      # experts 2 and 5 always tie: the lower id must win
    wg = rnd(1, width, dtype=torch.bfloat16, seed=2, scale=0.2) if with_gate else None
    ids = torch.empty(n, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, k, device=DEV)
    gate = torch.zeros(n, device=DEV)
    probs = torch.empty(n, e, device=DEV)
    logits = torch.empty(n, e + 1, device=DEV)
    st = status()
    ops.router_topk(h, wr, wg, ids, wts, gate, k, True, st, probs, logits=logits)
    assert st.item() == 0
    exact = h.double() @ wr.double().t()
    # a 32-bit dot product of `width` terms is good to about width * 2^-24 of the sum of magnitudes
    bound = (h.double().abs() @ wr.double().abs().t()) * (width * 2.0 ** -24)
    err = (logits[:, :e].double() - exact).abs()
    assert torch.all(err <= bound + 1e-30), f"logits off by {float((err / bound).max()):.2f} of the 32-bit bound"
    assert float((err / bound).max()) < 0.25, "the error should sit well inside the bound"
    p = torch.softmax(exact, -1)
    # a probability moves by at most p * (its own logit's error + the largest error of the row), plus float rounding
    p_err = (probs.double() - p).abs()
    p_bound = p * (bound + bound.max(-1, keepdim=True).values) + 4 * 2.0 ** -24
    assert torch.all(p_err <= p_bound), f"probabilities off by {float((p_err / p_bound).max()):.2f} of their bound"
    if with_gate:
        g_exact = (h.double() @ wg.double().t())[:, 0]
        g_bound = (h.double().abs() @ wg.double().abs().t())[:, 0] * (width * 2.0 ** -24)
        assert torch.all((logits[:, e].double() - g_exact).abs() <= g_bound)
        # the sigmoid's slope is at most 1/4
        assert torch.all((gate.double() - torch.sigmoid(g_exact)).abs() <= 0.25 * g_bound + 4 * 2.0 ** -24), "shared gate"
    pn, got = p.cpu().numpy(), ids.cpu().numpy()
    order = np.argsort(-pn, axis=1, kind="stable")[:, :k]
    for t in range(n):
        if list(got[t]) != list(order[t]):
            # only where two probabilities are closer than 32-bit arithmetic can tell may the choice differ
            a, b = sorted(set(got[t]) ^ set(order[t]))[:2] if set(got[t]) != set(order[t]) else (got[t][0], got[t][0])
            assert abs(pn[t, a] - pn[t, b]) <= 1e-6 * pn[t].max() or sorted(got[t]) == sorted(order[t]), (t, got[t], order[t])
        if e > 5:
            assert not (5 in got[t] and 2 not in got[t])


@pytest.mark.parametrize("n, k, e", [(1500, 3, 60), (700, 4, 7), (4096, 2, 64)])
def test_moe_permute_many_pairs_with_uneven_routing(n, k, e):
    """From 2,048 (token, expert) pairs on the permutation counts per warp; most tokens go to a few experts here
    and some experts get none.  Every pair must land exactly once inside its expert's range, and the tile list
    must cover the ranges without mixing experts."""
    rng = np.random.default_rng(n)
    p = rng.dirichlet(np.ones(e) * 0.15)
    ids_np = np.stack([rng.choice(e, size=k, replace=False, p=p / p.sum()) if np.count_nonzero(p) >= k else rng.permutation(e)[:k]
                       for _ in range(n)]).astype(np.int32)
    ids = torch.tensor(ids_np, device=DEV)
    wts = rnd(n, k).abs() + 0.01
    i32 = lambda *shape: torch.empty(*shape, dtype=torch.int32, device=DEV)
    offsets, perm_token, inverse = i32(e + 1), i32(n * k), i32(n, k)
    perm_weight = torch.empty(n * k, device=DEV)
    tile = ops.TC05_TILE_ROWS
    max_tiles = (n * k + tile - 1) // tile + e
    tiles = (i32(max_tiles), i32(max_tiles), i32(max_tiles), i32(1))
    st = status()
    ops.moe_permute(ids, wts, e, offsets, perm_token, perm_weight, inverse, st, tiles=tiles)
    assert st.item() == 0
    off = offsets.cpu().numpy()
    assert list(off) == list(np.concatenate([[0], np.cumsum(np.bincount(ids_np.reshape(-1), minlength=e))]))
    inv, pt, pw, w_np = inverse.cpu().numpy(), perm_token.cpu().numpy(), perm_weight.cpu().numpy(), wts.cpu().numpy()
    assert sorted(inv.reshape(-1)) == list(range(n * k)), "a row was given twice or not at all"
    rows = inv.reshape(-1)
    ex = ids_np.reshape(-1)
    assert np.all((off[ex] <= rows) & (rows < off[ex + 1])), "a pair outside its expert's range"
    assert np.array_equal(pt[rows], np.repeat(np.arange(n), k)) and np.array_equal(pw[rows], w_np.reshape(-1))
    n_tiles = tiles[3].item()
    tg, tr, tc = (t.cpu().numpy()[:n_tiles] for t in tiles[:3])
    assert n_tiles == sum((off[i + 1] - off[i] + tile - 1) // tile for i in range(e)) and sum(tc) == n * k
    assert all(off[g] <= r and r + c <= off[g + 1] and 0 < c <= tile for g, r, c in zip(tg, tr, tc))
    check_tile_cover(tr, tc, n * k, tile)


def test_a_bounded_wait_that_runs_out_sets_the_status_and_leaves_the_device_usable():
    """The waits inside the kernels poll a limited number of times.  Here one waits on a barrier that
    nothing completes, with a limit of a few thousand polls: the kernel reports it and returns, the
    engine turns the word into an error, and the next kernel runs as ever."""
    st = status()
    ops.wait_probe(4000, st)
    torch.cuda.synchronize()
    assert st.item() == 4
    x = torch.empty(3, 200, device=DEV)
    ok = status()
    ops.embed_gather(rnd(10, 200), torch.tensor([1, 2, 3], dtype=torch.int32, device=DEV), x, ok)
    assert ok.item() == 0 and torch.isfinite(x).all()


def test_attn_prefill_tc05_with_more_items_than_the_gpu_has_sms():
    """More (tile, head) items than the GPU has SMs, so that every persistent block of the tensor-memory
    prefill attention takes a second and third item with its rings and phases carried over."""
    check_attn_prefill(ops.attn_prefill_tc05, 24, 8, 128, None, tile=ops.ATTN_TC05_TILE_ROWS, runs=[
        (0, 900), (130, 700), (0, 1), (63, 66), (300, 129), (10, 420), (0, 384), (5, 250)])


@pytest.mark.parametrize("m, nh, nkv, hd, k", [(1, 4, 2, 128, 512), (8, 16, 16, 128, 2048), (13, 6, 3, 64, 384), (16, 7, 1, 32, 200)])
def test_qkv_projection_with_rotation_and_cache_write_in_one_kernel(m, nh, nkv, hd, k):
    """The fused kernel against the two kernels it replaces (same arithmetic in the same order: equal bits)
    and against a float64 restatement."""
    torch.manual_seed(4)
    width = (nh + 2 * nkv) * hd
    a = rnd(m, k, dtype=torch.bfloat16, scale=0.5)
    w = rnd(width, k, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias = rnd(width, scale=0.1, seed=2)
    max_pos, n_pages, half = 300, 9, hd // 2
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / (1e4 ** (torch.arange(half, dtype=torch.float64) * 2 / hd))[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    seqs = torch.arange(m, dtype=torch.int32, device=DEV) % 3
    pos = torch.tensor([(37 * i + 5) % max_pos for i in range(m)], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3 * p + s_ for p in range(5)] for s_ in range(3)], dtype=torch.int32, device=DEV) % n_pages
    table = torch.tensor([[0, 3, 6, 1, 4], [7, 2, 5, 8, 0], [4, 1, 8, 3, 6]], dtype=torch.int32, device=DEV)
    outs = []
    for fused in (False, True):
        q = torch.zeros(m, nh * hd, dtype=torch.bfloat16, device=DEV)
        kc = torch.zeros(n_pages, nkv, 64, hd, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        st = status()
        if fused:
            ops.qkv_rope_skinny(a, w, bias, seqs, pos, cos, sin, q, kc, vc, table, 64, nh, nkv, hd, True, st)
        else:
            qkv = torch.empty(m, width, device=DEV)
            ops.gemm_skinny(a, w, qkv)
            ops.rope_kvwrite(qkv, bias, seqs, pos, cos, sin, hd, q, kc, vc, table, 64, nh, nkv, hd, True, st)
        assert st.item() == 0
        outs.append((q, kc, vc))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    # float64: projection, bias, rotation of queries
    ref = a.double() @ w.double().t() + bias.double()
    qr = ref[:, :nh * hd].reshape(m, nh, hd)
    c, s_ = torch.cos(ang).to(DEV)[pos.long()][:, None, :], torch.sin(ang).to(DEV)[pos.long()][:, None, :]
    rot = torch.cat([qr[..., :half] * c - qr[..., half:] * s_, qr[..., half:] * c + qr[..., :half] * s_], -1)
    close(outs[1][0].view(m, nh, hd), rot, torch.bfloat16, "rotated queries", k=k)
