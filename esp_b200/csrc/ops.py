"""Python faces of the compiled kernels.

Every function here checks what it is given (device, dtype, contiguity, the
sizes the kernel takes), launches on torch's current stream and raises
``Backend`` if the launch is refused.  There is no other implementation behind
these functions: without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..errors import Backend
from .build import load_library

P = c_void_p

_SIGNATURES = {
    "esp_embed_gather": [P, c_int, P, P, c_int, c_int, c_int, c_float, P, P],
    "esp_softcap": [P, c_longlong, c_float, P],
    "esp_feed_tokens": [P, P, P, c_int, P],
    "esp_add_rmsnorm": [P, P, P, P, P, c_int, P, c_int, c_int, c_float, c_int, P],
    "esp_swiglu": [P, P, c_int, c_longlong, c_int, P],
    "esp_finite_check": [P, c_int, c_longlong, P, c_int, P],
    "esp_normal_fill": [P, c_int, c_longlong, c_ulonglong, c_float, c_float, P],
    "esp_gemm_simt": [P, c_int, P, P, c_int, P, P, P, c_int, P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, P],
    "esp_rope_kvwrite": [P, P, P, P, P, P, c_int, c_int, P, P, P, c_int, P, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_int, P, P],
    "esp_attn_simt": [P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_router_topk": [P, c_int, P, P, c_int, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_moe_permute": [P, P, c_int, c_int, c_int, P, P, P, P, P, P, P, P, c_int, c_int, P, P, P],
    "esp_gather_rows": [P, P, P, c_int, c_int, P],
    "esp_route_small": [P, c_int, P, P, c_int, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P,
                        c_int, P],
    "esp_gemm_tc05": [P, c_longlong, P, c_int, c_int, P, P, c_longlong, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, P, P],
    "esp_wait_probe": [c_int, P, P],
    "esp_moe_combine": [P, P, P, P, P, P, c_int, c_int, c_int, P],
    "esp_pick_tokens": [P, c_int, c_int, P, P, P, P, P, P],
    "esp_moe_combine_add_rmsnorm": [P, P, P, P, P, P, P, P, P, c_int, P, c_int, c_int, c_int, c_float, c_int, P],
    "esp_gemm_skinny": [P, c_longlong, P, P, c_longlong, P, P, c_int, c_longlong, P, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, P],
    "esp_qkv_rope_skinny": [P, c_longlong, P, P, P, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, P, P],
    "esp_attn_prefill": [P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P],
    "esp_attn_prefill_tc05": [P, c_longlong, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              P, P],
    "esp_attn_decode": [P, P, P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int, P, P],
}

_bound: dict = {}


def _fn(library: str, name: str):
    f = _bound.get(name)
    if f is None:
        lib = load_library(library)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise Backend(f"the compiled library '{library}' has no entry point {name}") from None
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _bound[name] = f
    return f


_device_index = None


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so it takes the short way (the full
    ``torch.cuda.current_stream()`` costs several microseconds a call, a quarter of an eager step's host time)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(_device_index)
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Kernel launches made through this module since the process started."""
    return _launches


def add_launches(count: int) -> None:
    """Accounts for kernels that ran through the replay of a captured graph."""
    global _launches
    _launches += count


class LaunchProfile:
    """Device time by kind of kernel.  While one is active (``with LaunchProfile() as prof``) every launch made
    through this module on the current stream is followed by a CUDA event; the time between two events is
    charged to the later launch (so a launch's share holds the gap before it as well).  Meant for steps that
    run eagerly on one stream: no captured graphs, nothing on a second stream."""

    active = None

    def __init__(self):
        self.marks = []                      # (what, event)

    def __enter__(self):
        first = torch.cuda.Event(enable_timing=True)
        first.record()
        self.marks = [("start", first)]
        LaunchProfile.active = self
        return self

    def __exit__(self, *exc):
        LaunchProfile.active = None

    def note(self, what: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((what, ev))

    def rows(self) -> list:
        """[(kind, launches, microseconds)], the largest first."""
        torch.cuda.synchronize()
        total: dict = {}
        for (_w0, e0), (what, e1) in zip(self.marks, self.marks[1:]):
            n, us = total.get(what, (0, 0.0))
            total[what] = (n + 1, us + e0.elapsed_time(e1) * 1e3)
        return sorted(((w, n, us) for w, (n, us) in total.items()), key=lambda r: -r[2])

    def table(self) -> str:
        rows = self.rows()
        whole = sum(us for _w, _n, us in rows) or 1.0
        lines = [f"{'kernel':<28}{'launches':>9}{'us':>12}{'share':>8}"]
        lines += [f"{w:<28}{n:>9}{us:>12.1f}{us / whole:>8.1%}" for w, n, us in rows]
        lines.append(f"{'all':<28}{sum(n for _w, n, _u in rows):>9}{whole:>12.1f}{1:>8.0%}")
        return "\n".join(lines)


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if LaunchProfile.active is not None:
        LaunchProfile.active.note(what)
    if code != 0:
        raise Backend(f"{what}: the launch was refused with CUDA error {code} "
                      f"(invalid value means a size this kernel does not take)")


def _ptr(t, dtype=None, what="tensor"):
    if t is None:
        return None
    if not t.is_cuda:
        raise Backend(f"{what} must live on the GPU; this library has no CPU path")
    if not t.is_contiguous():
        raise Backend(f"{what} must be contiguous")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise Backend(f"{what} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


FLOATS = (torch.float32, torch.bfloat16)


def _is_bf16(t) -> int:
    return 1 if t.dtype == torch.bfloat16 else 0


# ---------------------------------------------------------------------------

def embed_gather(table, ids, x, status, scale: float = 1.0):
    """x[n] = scale * float(table[ids[n]]); ids int32 [N], x float32 [N, H]."""
    n, width = x.shape
    _check(_fn("core", "esp_embed_gather")(
        _ptr(table, FLOATS, "embedding table"), _is_bf16(table), _ptr(ids, torch.int32, "ids"),
        _ptr(x, torch.float32, "x"), n, width, table.shape[0], float(scale), _ptr(status, torch.int32), _stream()),
        "embed_gather")


def softcap(values, cap: float):
    """values = cap * tanh(values / cap), in place (float32)."""
    if not cap > 0:
        raise Backend(f"softcap: the cap must be positive, got {cap}")
    _check(_fn("core", "esp_softcap")(_ptr(values, torch.float32, "values"), values.numel(), float(cap), _stream()),
           "softcap")


def feed_tokens(ids, picks, src):
    """ids[j] = picks[src[j]] where src[j] >= 0 (all int32 on the device)."""
    _check(_fn("core", "esp_feed_tokens")(_ptr(ids, torch.int32, "ids"), _ptr(picks, torch.int32, "picks"),
                                           _ptr(src, torch.int32, "src"), ids.shape[0], _stream()), "feed_tokens")


def add_rmsnorm(x, y, gamma, h, eps, rows=None, write_x=True, h32=None):
    """h = rmsnorm(x + y) * gamma with x (+= y when write_x) float32, gamma
    float32, h float32 or bfloat16.  ``rows`` (int32) selects source rows;
    ``h32`` (float32, same shape as h) receives the unrounded rows."""
    n_rows = h.shape[0]
    width = h.shape[1]
    if x.shape[1] != width or gamma.shape[0] != width:
        raise Backend("add_rmsnorm: widths disagree")
    _check(_fn("core", "esp_add_rmsnorm")(
        _ptr(x, torch.float32, "x"), _ptr(y, torch.float32, "y"), _ptr(gamma, torch.float32, "gamma"),
        _ptr(rows, torch.int32, "rows"), _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(h32, torch.float32, "h32"), n_rows,
        width, float(eps),
        1 if write_x else 0, _stream()), "add_rmsnorm")


def swiglu(gu, act):
    """act[m, i] = silu(gu[m, i]) * gu[m, I + i]; gu float32 [M, 2I]."""
    rows, inter = act.shape
    if gu.shape[0] < rows or gu.shape[1] != 2 * inter:
        raise Backend("swiglu: gu must be [rows, 2 * intermediate]")
    _check(_fn("core", "esp_swiglu")(_ptr(gu, torch.float32, "gu"), _ptr(act, FLOATS, "act"), _is_bf16(act), rows,
                                     inter, _stream()), "swiglu")


STATUS_LOGITS_NONFINITE = 2


def finite_check(values, status, bit: int = STATUS_LOGITS_NONFINITE):
    """ORs ``bit`` into status[0] if ``values`` (float32 or bfloat16, contiguous) hold a NaN or an infinity."""
    _check(_fn("core", "esp_finite_check")(_ptr(values, FLOATS, "values"), _is_bf16(values), values.numel(),
                                           _ptr(status, torch.int32), int(bit), _stream()), "finite_check")


def normal_fill(out, key: int, mean: float, std: float):
    """out[i] = mean + std * z(key, i), z standard normal, counter-based."""
    _check(_fn("core", "esp_normal_fill")(_ptr(out, FLOATS, "out"), _is_bf16(out), out.numel(),
                                          key & 0xFFFFFFFFFFFFFFFF, float(mean), float(std), _stream()), "normal_fill")


def gemm_simt(a, w, c, bias=None, row_scale=None, a_rows=None, group_offsets=None, rows=None):
    """c[m, :] = (a[a_rows[m] or m, :] @ w[g].T + bias) * row_scale[m] with true
    32-bit multiply-adds.  ``w`` is [N, K] or, grouped, [G, N, K] with
    ``group_offsets`` int32 [G+1] over the rows.  ``rows``: how many rows of c to
    compute (default: all of c)."""
    grouped = group_offsets is not None
    if grouped:
        groups, n, k = w.shape
    else:
        groups = 1
        n, k = w.shape
    m = c.shape[0] if rows is None else rows
    if a.shape[-1] != k or c.shape[-1] != n:
        raise Backend(f"gemm: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    if a.stride(-1) != 1 or c.stride(-1) != 1 or not w.is_contiguous():
        raise Backend("gemm: operands must be row-major")
    code = _fn("core", "esp_gemm_simt")(
        a.data_ptr(), _is_bf16(a), _ptr(a_rows, torch.int32, "a_rows"), w.data_ptr(), _is_bf16(w),
        _ptr(bias, torch.float32, "bias"), _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(), _is_bf16(c),
        _ptr(group_offsets, torch.int32, "group_offsets"), groups, m, n, k, a.stride(0), c.stride(0), _stream())
    _check(code, "gemm_simt")


def rope_kvwrite(qkv, bias, tok_seq, tok_pos, cos, sin, rot, q_out, k_cache, v_cache, block_table, page, nh, nkv, hd,
                 write_kv, status):
    """Add the bias, rotate queries and keys (split-half, 32-bit) and store keys
    and values in the paged cache.  k_cache/v_cache: [pages, nkv, page, hd]."""
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise Backend("rope_kvwrite: qkv width disagrees with the head counts")
    n_pages = k_cache.shape[0] if k_cache is not None else 0
    _check(_fn("core", "esp_rope_kvwrite")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(bias, torch.float32, "bias"), _ptr(tok_seq, torch.int32),
        _ptr(tok_pos, torch.int32), _ptr(cos, torch.float32), _ptr(sin, torch.float32), rot, cos.shape[0] if cos is not None else (1 << 30),
        _ptr(q_out, FLOATS, "q_out"), _ptr(k_cache, FLOATS), _ptr(v_cache, FLOATS), _is_bf16(q_out),
        _ptr(block_table, torch.int32), block_table.shape[1] if block_table is not None else 0, n_pages, page, n,
        nh, nkv, hd, 1 if write_kv else 0, _ptr(status, torch.int32), _stream()), "rope_kvwrite")


def attn_simt(q, k_cache, v_cache, out, tok_seq, tok_pos, block_table, page, nh, nkv, hd, window, status):
    """Attention of every token over its sequence's cached keys (32-bit arithmetic)."""
    if hd > 256:
        raise Backend(f"attention: head size {hd} is beyond the 256 this kernel takes")
    _check(_fn("core", "esp_attn_simt")(
        _ptr(q, FLOATS, "q"), _ptr(k_cache, FLOATS), _ptr(v_cache, FLOATS), _ptr(out, FLOATS), _is_bf16(q),
        _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(block_table, torch.int32), block_table.shape[1],
        k_cache.shape[0], page, q.shape[0], nh, nkv, hd, int(window or 0), _ptr(status, torch.int32), _stream()),
        "attn_simt")


def router_topk(h, w_router, w_gate, topk_ids, topk_w, gate, top_k, norm_topk, status, probs_out=None, logits=None):
    """``logits``: optional float32 scratch [n, experts + 1]; with it, 32-bit activations and bfloat16 weights
    the logits of a step of many tokens are made on the tensor cores (three bfloat16 parts of every
    activation: products exact, sums in float)."""
    n, width = h.shape
    n_experts = w_router.shape[0]
    if top_k > 32:
        raise Backend(f"router: top-k {top_k} is beyond the 32 this kernel takes")
    if (width + n_experts) * 4 > 200 * 1024:
        raise Backend(f"router: width {width} + experts {n_experts} do not fit the kernel's shared memory")
    if w_gate is not None and w_gate.dtype != w_router.dtype:
        raise Backend("router: router and shared-gate weights must share a dtype")
    if logits is not None and logits.numel() < n * (n_experts + 1):
        raise Backend("router: the logits scratch is smaller than [tokens, experts + 1]")
    _check(_fn("core", "esp_router_topk")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(w_router, FLOATS), _ptr(w_gate, FLOATS), _is_bf16(w_router),
        _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32), _ptr(gate, torch.float32),
        _ptr(probs_out, torch.float32), _ptr(logits, torch.float32), n, width, n_experts, top_k, 1 if norm_topk else 0,
        _ptr(status, torch.int32), _stream()), "router_topk")


ROUTE_SMALL_TOKENS = 64


def route_small_fits(width: int, n_experts: int) -> bool:
    # the second kernel's shared memory: probabilities of eight tokens, counts and cursors, and the step's pairs
    return width * 4 <= 48 * 1024 and (8 * n_experts) * 4 + (2 * n_experts + 1) * 4 + ROUTE_SMALL_TOKENS * 32 * 8 <= 48 * 1024


def route_small(h, w_router, w_gate, logits, topk_ids, topk_w, gate, top_k, norm_topk, offsets, perm_token,
                perm_weight, inverse, status, probs_out=None, distinct=None, tiles=None):
    """Router and permutation for at most ROUTE_SMALL_TOKENS tokens: logits over many blocks, then one
    block for softmax, top-k and the permutation.  ``logits``: float32 scratch [N, E + 1].  ``distinct``:
    an int64 tensor of one element to which the number of experts with at least one token is added.
    ``tiles``: as for moe_permute (the row tiles of the grouped tensor-core products; one per expert with rows)."""
    n, width = h.shape
    n_experts = w_router.shape[0]
    if n > ROUTE_SMALL_TOKENS or top_k > 32 or not route_small_fits(width, n_experts):
        raise Backend("route_small: too many tokens or experts for this kernel")
    _check(_fn("core", "esp_route_small")(
        _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(w_router, FLOATS), _ptr(w_gate, FLOATS), _is_bf16(w_router),
        _ptr(logits, torch.float32), _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32),
        _ptr(gate, torch.float32), _ptr(probs_out, torch.float32), n, width, n_experts, top_k, 1 if norm_topk else 0,
        _ptr(offsets, torch.int32), _ptr(perm_token, torch.int32), _ptr(perm_weight, torch.float32),
        _ptr(inverse, torch.int32), _ptr(status, torch.int32), _ptr(distinct, torch.int64),
        _ptr(tiles[0], torch.int32) if tiles else None, _ptr(tiles[1], torch.int32) if tiles else None,
        _ptr(tiles[2], torch.int32) if tiles else None, _ptr(tiles[3], torch.int32) if tiles else None,
        tiles[0].shape[0] if tiles else 0, _stream()), "route_small")


def moe_permute(topk_ids, topk_w, n_experts, offsets, perm_token, perm_weight, inverse, status, tiles=None,
                distinct=None):
    """``distinct``: as for route_small.  ``tiles``: optional (tile_group, tile_row0, tile_count, n_tiles) int32 tensors that receive the
    list of row tiles (of at most TC05_TILE_ROWS rows) for the grouped tensor-core products."""
    n, top_k = topk_ids.shape
    if (2 * n_experts + 1) * 4 > 48 * 1024:
        raise Backend(f"moe_permute: {n_experts} experts are beyond what this kernel takes")
    _check(_fn("core", "esp_moe_permute")(
        _ptr(topk_ids, torch.int32), _ptr(topk_w, torch.float32), n, top_k, n_experts, _ptr(offsets, torch.int32),
        _ptr(perm_token, torch.int32), _ptr(perm_weight, torch.float32), _ptr(inverse, torch.int32),
        _ptr(tiles[0], torch.int32) if tiles else None, _ptr(tiles[1], torch.int32) if tiles else None,
        _ptr(tiles[2], torch.int32) if tiles else None, _ptr(tiles[3], torch.int32) if tiles else None,
        TC05_TILE_ROWS if tiles else 0, tiles[0].shape[0] if tiles else 0, _ptr(status, torch.int32),
        _ptr(distinct, torch.int64), _stream()), "moe_permute")


def moe_combine(expert_out, topk_ids, inverse, gate, shared, y):
    n, width = y.shape
    _check(_fn("core", "esp_moe_combine")(
        _ptr(expert_out, torch.float32), _ptr(topk_ids, torch.int32), _ptr(inverse, torch.int32),
        _ptr(gate, torch.float32), _ptr(shared, torch.float32), _ptr(y, torch.float32), n, width, topk_ids.shape[1],
        _stream()), "moe_combine")


def moe_combine_add_rmsnorm(expert_out, topk_ids, inverse, gate, shared, x, gamma, h, eps, rows=None, write_x=True,
                            h32=None):
    """moe_combine followed by add_rmsnorm in one kernel (same operations in the same order): x (+)= combined
    expert outputs, h = rmsnorm(x) * gamma.  Width a multiple of 4, at most 16384."""
    n_rows, width = h.shape
    if width % 4 != 0 or width > 16384:
        raise Backend(f"moe_combine_add_rmsnorm: width {width} not taken")
    _check(_fn("core", "esp_moe_combine_add_rmsnorm")(
        _ptr(expert_out, torch.float32), _ptr(topk_ids, torch.int32), _ptr(inverse, torch.int32),
        _ptr(gate, torch.float32), _ptr(shared, torch.float32), _ptr(x, torch.float32), _ptr(gamma, torch.float32),
        _ptr(rows, torch.int32), _ptr(h, FLOATS, "h"), _is_bf16(h), _ptr(h32, torch.float32), n_rows, width,
        topk_ids.shape[1], float(eps), 1 if write_x else 0, _stream()), "moe_combine_add_rmsnorm")


def pick_tokens(logits, temperature, top_p, rng_state, row_slot, tokens):
    """tokens[r] = arg-max of row r when temperature[r] == 0 (or temperature is
    None), else a draw from the row's own splitmix64 stream rng_state[row_slot[r]]
    (int64 storage read as unsigned)."""
    n, vocab = logits.shape
    _check(_fn("core", "esp_pick_tokens")(
        _ptr(logits, torch.float32, "logits"), n, vocab, _ptr(temperature, torch.float32), _ptr(top_p, torch.float32),
        _ptr(rng_state, torch.int64), _ptr(row_slot, torch.int32), _ptr(tokens, torch.int32), _stream()), "pick_tokens")


# ---------------------------------------------------------------------------
# bfloat16 kernels (library "bf16")
# ---------------------------------------------------------------------------
SKINNY_MAX_SMEM = 227 * 1024


def skinny_fits(k: int) -> bool:
    """Whether gemm_skinny can stage eight activation rows of width k."""
    return k % 8 == 0 and 8 * (k + 32) * 2 + 8 * 512 <= SKINNY_MAX_SMEM


def gemm_skinny(a, w, c, swiglu=False, row_scale=None, a_rows=None, group_offsets=None, rows=None, max_rows=None,
                offsets_ready=False):
    """Weight-streaming product for few rows; bfloat16 a and w.  Plain: c[m] =
    scale[m] * a[row(m)] @ w[g].T with w [N,K] or [G,N,K].  swiglu: w holds
    [gate rows; up rows] ([2I,K] or [G,2I,K]) and c[m, j] = silu(gate_j) * up_j
    ([rows, I]).  ``max_rows``: upper bound of the rows of one group.  ``offsets_ready``: the group offsets (and
    ``row_scale``) were complete before the kernel that runs right before this one started, so this one may
    find its group and ask for its weights while that kernel still runs (only ``a`` is waited for)."""
    grouped = group_offsets is not None
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise Backend("gemm_skinny takes bfloat16 operands")
    if grouped:
        groups, wn, k = w.shape
    else:
        groups = 1
        wn, k = w.shape
    n = wn // 2 if swiglu else wn
    m = c.shape[0] if rows is None else rows
    if a.shape[-1] != k or c.shape[-1] != n or a.stride(-1) != 1 or c.stride(-1) != 1 or not w.is_contiguous():
        raise Backend(f"gemm_skinny: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    if k % 8 != 0 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        raise Backend(f"gemm_skinny: width {k} (and the row stride) must be a multiple of 8")
    if max_rows is None:
        max_rows = m
    code = _fn("bf16", "esp_gemm_skinny")(
        a.data_ptr(), a.stride(0), _ptr(a_rows, torch.int32, "a_rows"), w.data_ptr(), wn * k,
        _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(), _is_bf16(c), c.stride(0),
        _ptr(group_offsets, torch.int32, "group_offsets"), groups, m, n, k, max_rows, 1 if swiglu else 0,
        1 if offsets_ready else 0, _stream())
    _check(code, "gemm_skinny")


def qkv_rope_skinny_fits(rows: int, k: int, hd: int) -> bool:
    return rows <= 16 and hd % 16 == 0 and skinny_fits(k)


def qkv_rope_skinny(a, w_qkv, bias, tok_seq, tok_pos, cos, sin, q_out, k_cache, v_cache, block_table, page, nh, nkv, hd,
                    write_kv, status):
    """The packed q/k/v projection of at most 16 rows with bias, full split-half rotation of queries and keys
    and the cache write in one kernel (bfloat16): what gemm_skinny followed by rope_kvwrite computes."""
    m, k = a.shape
    if w_qkv.shape != ((nh + 2 * nkv) * hd, k) or not qkv_rope_skinny_fits(m, k, hd):
        raise Backend(f"qkv_rope_skinny: sizes not taken: a {tuple(a.shape)}, w {tuple(w_qkv.shape)}, head size {hd}")
    if cos.shape[1] != hd // 2:
        raise Backend("qkv_rope_skinny rotates the whole head: the tables must be [positions, head size / 2]")
    if a.stride(-1) != 1 or a.stride(0) % 8 != 0 or a.data_ptr() % 16 != 0:
        raise Backend("qkv_rope_skinny: the rows must be 16-byte aligned")
    _check(_fn("bf16", "esp_qkv_rope_skinny")(
        _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else a.data_ptr(), a.stride(0), _ptr(w_qkv, torch.bfloat16, "w_qkv"),
        _ptr(bias, torch.float32, "bias"), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32),
        _ptr(cos, torch.float32, "cos"), _ptr(sin, torch.float32, "sin"), cos.shape[0], _ptr(q_out, torch.bfloat16, "q_out"),
        _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, m, k, nh, nkv, hd, 1 if write_kv else 0,
        _ptr(status, torch.int32), _stream()), "qkv_rope_skinny")


# blocks of the split-key kernel that one SM holds at a time, by head size (registers: 72 / 122 / 160 / 162 a thread)
ATTN_DECODE_BLOCKS_PER_SM = {64: 7, 128: 4, 192: 3, 256: 3}


@functools.lru_cache(maxsize=4096)
def attn_decode_split(n_rows: int, nkv_blocks: int, positions: int, head_dim: int = 128, sm_count: int = 148) -> int:
    """Key positions per block (whole pages of 64), the same for every row of the step: the length with the least
    estimated time.  The estimate, fitted to steps of 1 to 64 rows with 16 key/value heads of 128 at 4,096
    positions and checked at 8,000 to 32,000 positions with 4: the device holds ``room`` blocks at once and needs
    three quarters of that many to draw the full memory rate; blocks start as others end, so the time is that of
    all blocks' pages at the full rate, plus what the last, partly filled round lacks of three quarters, plus one
    page's time a block for its start, its partial result and its share of the combine.  It gives one round of
    short blocks to a few rows (128 positions at batch 1, 256 at batch 2, 1,024 at batch 8), whole rows to 32 or
    64 rows, and thirds or quarters of a row where whole rows would leave a round nearly empty (batch 24, 40, 48).
    Against the earlier choice among 128, 256 and 512 under a limit of 1,024 blocks: batch 2 +3.5 %, 5 +6 %, 6 +5 %,
    8 +1.5 %, 16 +4 %, 32 +4 %, 48 +2 %, 64 +4.5 %; batch 8 at 8,000 positions +5 %.  At least 128 positions, 256 beyond
    4,096 (at batch 1, 128 gains 1 % at 4,096 positions and loses 7 % at 8,192 with 4 key/value heads)."""
    room = sm_count * ATTN_DECODE_BLOCKS_PER_SM.get(head_dim, 3)
    full_rate = 0.75 * room
    pairs = max(1, n_rows * nkv_blocks)
    pages = max(1, (positions + 63) // 64)
    shortest = min(pages, 2 if positions <= 4096 else 4)
    best, best_cost = pages, None
    for length in range(pages, shortest - 1, -1):          # longest first: it wins a tie
        blocks = pairs * ((pages + length - 1) // length)
        last = blocks % room
        cost = (blocks + (full_rate - last if 0 < last < full_rate else 0.0)) * (length + 1.0)
        if best_cost is None or cost < best_cost:
            best, best_cost = length, cost
    return 64 * best


ATTN_DECODE_COUNTERS = 65536


def attn_decode(q, k_cache, v_cache, out, part_o, part_ml, counters, tok_seq, tok_pos, block_table, page, nh, nkv, hd,
                window, split, n_splits, status, seq_past=None):
    """Split-key attention for few token rows (bfloat16; head sizes 64, 128, 192, 256).  ``split``: key
    positions per block (a multiple of 64); n_splits >= ceil(positions / split).  part_o float32
    [N, nh, n_splits, hd] and part_ml float32 [N, nh, n_splits, 2] are scratch; ``counters``: int32, at least
    N * nh words, all zero (the kernel leaves them zero).  ``seq_past`` (int32 per sequence of the step: the
    positions cached before it): blocks whose keys are all older then load them without waiting for the
    kernel before this one, which writes the step's new keys and values."""
    if counters.numel() < q.shape[0] * nh:
        raise Backend("attn_decode: too few counters for this many rows and heads")
    if split < 64 or split % 64:
        raise Backend(f"attn_decode: split {split} is not a multiple of 64")
    if hd not in (64, 128, 192, 256):
        raise Backend(f"attn_decode: head size {hd} is not one of 64, 128, 192, 256")
    n = q.shape[0]
    if part_o.numel() < n * nh * n_splits * hd or part_ml.numel() < n * nh * n_splits * 2:
        raise Backend("attn_decode: scratch is too small")
    _check(_fn("bf16", "esp_attn_decode")(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(part_o, torch.float32), _ptr(part_ml, torch.float32),
        _ptr(counters, torch.int32), _ptr(tok_seq, torch.int32), _ptr(tok_pos, torch.int32), _ptr(seq_past, torch.int32),
        _ptr(block_table, torch.int32), block_table.shape[1],
        k_cache.shape[0], page, n, nh, nkv, hd, int(window or 0), split, n_splits, _ptr(status, torch.int32),
        _stream()), "attn_decode")


def attn_prefill(q, k_cache, v_cache, out, tile_seq, tile_first, seq_start, seq_past, block_table, page, nh, nkv, hd,
                 window, status):
    """Flash-style attention for runs of new tokens (bfloat16; head sizes that are multiples of 8 up to
    128; pages of 64 positions).  tile_seq / tile_first describe the tiles of 64 new tokens."""
    if hd % 8 != 0 or hd > 128 or page != 64:
        raise Backend(f"attn_prefill: head size {hd} / page {page} not taken (multiples of 8 up to 128; page 64)")
    _check(_fn("bf16", "esp_attn_prefill")(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(tile_seq, torch.int32), _ptr(tile_first, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_past, torch.int32), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, tile_seq.shape[0], nh, nkv, hd, int(window or 0),
        _ptr(status, torch.int32), _stream()), "attn_prefill")


ATTN_TC05_TILE_ROWS = 128      # new tokens of a sequence to a tile of attn_prefill_tc05


def attn_prefill_tc05_fits(hd, page) -> bool:
    """Head sizes and page size that the tensor-memory prefill attention takes."""
    return hd in (64, 128) and page == 64


def attn_prefill_tc05(q, k_cache, v_cache, out, tile_seq, tile_first, seq_start, seq_past, block_table, page, nh, nkv, hd,
                      window, status):
    """Prefill attention on tcgen05 with accumulators in tensor memory (bfloat16; head size 64 or 128; pages
    of 64 positions).  Same arguments as attn_prefill, but tile_seq / tile_first list tiles of
    ATTN_TC05_TILE_ROWS new tokens, best with the tiles that see the most keys first (the order only matters
    for the balance)."""
    if not attn_prefill_tc05_fits(hd, page):
        raise Backend(f"attn_prefill_tc05: head size {hd} / page {page} not taken (64 or 128; page 64)")
    if not q.is_contiguous() or q.numel() != q.shape[0] * nh * hd:
        raise Backend("attn_prefill_tc05 takes contiguous queries [tokens, heads * head size]")
    _check(_fn("tc05", "esp_attn_prefill_tc05")(
        _ptr(q, torch.bfloat16, "q"), q.shape[0], _ptr(k_cache, torch.bfloat16), _ptr(v_cache, torch.bfloat16),
        _ptr(out, torch.bfloat16), _ptr(tile_seq, torch.int32), _ptr(tile_first, torch.int32),
        _ptr(seq_start, torch.int32), _ptr(seq_past, torch.int32), _ptr(block_table, torch.int32),
        block_table.shape[1], k_cache.shape[0], page, tile_seq.shape[0], nh, nkv, hd, int(window or 0),
        _ptr(status, torch.int32), _stream()), "attn_prefill_tc05")


def gather_rows(src, rows, out):
    """out[r] = src[rows[r]] for bfloat16 rows (width a multiple of 8)."""
    _check(_fn("core", "esp_gather_rows")(_ptr(src, torch.bfloat16, "src"), _ptr(rows, torch.int32, "rows"),
                                          _ptr(out, torch.bfloat16, "out"), out.shape[0], src.shape[1], _stream()),
           "gather_rows")


TC05_TILE_ROWS = 256


# Which tensor-memory products run on pairs of CTAs (tcgen05 cta_group::2: one MMA of 256 weight rows, each CTA of
# the pair loads its own 128 and half of the token rows): "0" none, "grouped", "dense" or "all".  Measured at the
# A2.7B sizes, 2,048 tokens: grouped gate/up 143.5 -> 133.8 us, grouped down 86.9 -> 82.8 us, dense fused SwiGLU
# 78.4 -> 74.7 us, dense plain 42.3 -> 43.9 us; results are equal bit for bit.
TC05_PAIR = os.environ.get("ESP_B200_TC05_PAIR", "all")
TC05_PAIR_ROWS_PER_GROUP = 32          # grouped products with fewer rows per group than this run on single CTAs


def gemm_tc05(a, w, c, status, swiglu=False, row_scale=None, tiles=None, rows=None, tile_rows=None, pair=None,
              max_ctas=0):
    """TMA + tcgen05 product for many rows.  a [rows, K] bfloat16 contiguous; w [N, K] or [G, N, K]
    bfloat16.  Plain: c float32 [rows, N] = scale * a @ w[g].T.  swiglu: w rows are [gate; up] and c is
    bfloat16 [rows, I].  Grouped: ``tiles`` = (tile_group, tile_row0, tile_count, n_tiles) from moe_permute,
    ``tile_rows`` the most rows a tile has (128 or 256; TC05_TILE_ROWS when not given).  ``max_ctas`` > 0:
    the kernel takes at most that many SMs, so that kernels of another stream find room beside it."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not a.is_contiguous() or not w.is_contiguous():
        raise Backend("gemm_tc05 takes contiguous bfloat16 operands")
    if w.dim() == 3:
        groups, wn, k = w.shape
    else:
        groups = 1
        wn, k = w.shape
    n = wn // 2 if swiglu else wn
    m = a.shape[0] if rows is None else rows
    if a.shape[1] != k or c.shape[1] != n or k % 8 != 0 or c.stride(1) != 1:
        raise Backend(f"gemm_tc05: shapes disagree or K is no multiple of 8: a {tuple(a.shape)}, w {tuple(w.shape)}, "
                      f"c {tuple(c.shape)}")
    if c.dtype != (torch.bfloat16 if swiglu else torch.float32):
        raise Backend("gemm_tc05: the plain product writes float32, the SwiGLU product bfloat16")
    grouped = tiles is not None
    tile_rows = TC05_TILE_ROWS if tile_rows is None else tile_rows
    if pair is None:
        pair = TC05_PAIR == "all" or TC05_PAIR == ("grouped" if grouped else "dense")
        # narrow token tiles gain nothing from sharing them between two CTAs, and one MMA thread per CTA issues
        # more per SM than one per pair: a prompt of 256 tokens (17 rows an expert) 7.45 -> 6.91 ms on single
        # CTAs, one of 1,024 tokens (68 rows an expert) 8.11 -> 8.55 ms
        if grouped and m < TC05_PAIR_ROWS_PER_GROUP * groups:
            pair = False
    code = _fn("tc05", "esp_gemm_tc05")(
        a.data_ptr(), m, w.data_ptr(), groups, wn, _ptr(row_scale, torch.float32, "row_scale"), c.data_ptr(),
        c.stride(0), _ptr(tiles[0], torch.int32) if grouped else None,
        _ptr(tiles[1], torch.int32) if grouped else None, _ptr(tiles[2], torch.int32) if grouped else None,
        _ptr(tiles[3], torch.int32) if grouped else None, tiles[0].shape[0] if grouped else 0,
        tile_rows if grouped else 0, m, n, k,
        1 if swiglu else 0, 1 if pair else 0, int(max_ctas), _ptr(status, torch.int32), _stream())
    _check(code, "gemm_tc05")


def wait_probe(polls: int, status):
    """Runs the library's bounded wait on a barrier that nothing completes: after ``polls`` tries the
    kernel sets the wait-expired bit of ``status`` and returns."""
    _check(_fn("tc05", "esp_wait_probe")(int(polls), _ptr(status, torch.int32, "status"), _stream()), "wait_probe")
