"""The no-allocation entry point of the decode attention, called through its exported C symbol.

Some programs that embed the library cannot allocate device memory when they need attention: they gave
the whole device to their own arena at start-up, or they sit in a loop where cudaMalloc and cudaFree are
not allowed because either may wait for the device.  For them ``esp_attn_decode_noalloc`` keeps the
kernel's scratch in a fixed array inside the library.  This test calls the symbol twice in a row, with
different shapes so that the second call finds the first call's leftovers in the array, and compares
each result with the ordinary entry point's, which gets its scratch from the caller.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from esp_b200.csrc import ops
from esp_b200.csrc.build import load_library

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE = -2
SPLIT = 256          # key positions per block; the entry point takes any multiple of 64


def bind():
    lib = load_library("bf16")
    fn = lib.esp_attn_decode_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, P]
    fn.restype = I
    cap = lib.esp_attn_decode_noalloc_capacity
    cap.argtypes, cap.restype = [], ctypes.c_longlong
    return fn, cap


def case(seed, n_seq, nh, nkv, hd, max_len, window):
    """Random queries over a random paged cache: (tensors..., n_splits)."""
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = (max_len + 63) // 64
    n_pages = n_seq * pages_per_seq + 3
    k = (torch.randn(n_pages, nkv, 64, hd, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    v = torch.randn(n_pages, nkv, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    q = (torch.randn(n_seq, nh * hd, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(n_pages, generator=g)[:n_seq * pages_per_seq].reshape(n_seq, pages_per_seq)
    table = perm.to(torch.int32).to(DEV).contiguous()
    lens = torch.randint(1, max_len + 1, (n_seq,), generator=g)
    lens[0] = max_len
    pos = (lens - 1).to(torch.int32).to(DEV)
    seq = torch.arange(n_seq, dtype=torch.int32, device=DEV)
    n_splits = (pages_per_seq * 64 + SPLIT - 1) // SPLIT
    return q, k, v, seq, pos, table, n_splits, (nh, nkv, hd, window)


def run_both(fn, c):
    q, k, v, seq, pos, table, n_splits, (nh, nkv, hd, window) = c
    n = q.shape[0]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    part_o = torch.full((n, nh, n_splits, hd), float("nan"), device=DEV)
    part_ml = torch.full((n, nh, n_splits, 2), float("nan"), device=DEV)
    counters = torch.zeros(n * nh, dtype=torch.int32, device=DEV)
    ops.attn_decode(q, k, v, ref, part_o, part_ml, counters, seq, pos, table, 64, nh, nkv, hd, window, SPLIT, n_splits,
                    status)
    out = torch.full_like(ref, float("nan"))
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), seq.data_ptr(), pos.data_ptr(), table.data_ptr(),
            table.shape[1], k.shape[0], 64, n, nh, nkv, hd, window or 0, SPLIT, n_splits, status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0, f"esp_attn_decode_noalloc returned {rc}"
    assert status.item() == 0
    return out, ref


def plain_attention(c):
    """The same attention in float64 straight from the pages: query row i sees keys 0..pos[i] of its own
    sequence (the newest ``window`` of them when there is a window)."""
    q, k, v, seq, pos, table, _n_splits, (nh, nkv, hd, window) = c
    group = nh // nkv
    out = torch.zeros(q.shape[0], nh, hd, dtype=torch.float64)
    kd, vd, tab = k.double().cpu(), v.double().cpu(), table.cpu()
    for i in range(q.shape[0]):
        p = int(pos[i])
        lo = max(0, p - window + 1) if window else 0
        pages = tab[int(seq[i])]
        keys = torch.stack([kd[pages[j // 64], :, j % 64] for j in range(lo, p + 1)])      # [len, nkv, hd]
        vals = torch.stack([vd[pages[j // 64], :, j % 64] for j in range(lo, p + 1)])
        for h in range(nh):
            s = keys[:, h // group] @ q[i].double().cpu().view(nh, hd)[h] / np.sqrt(hd)
            out[i, h] = torch.softmax(s, 0) @ vals[:, h // group]
    return out.view(q.shape[0], nh * hd)


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    fn, cap = bind()
    assert cap() == (2 << 20) - 65536
    first = case(1, n_seq=6, nh=8, nkv=2, hd=128, max_len=900, window=None)
    second = case(2, n_seq=3, nh=4, nkv=4, hd=64, max_len=300, window=100)     # smaller: stale values stay beside it
    for c in (first, second):
        out, ref = run_both(fn, c)
        # the same kernel with the same splits in the same order: nothing but the scratch's address differs
        assert torch.equal(out, ref), "the result depends on where the scratch lies"
        want = plain_attention(c)
        scale = float(want.abs().max())
        err = float((out.double().cpu() - want).abs().max())
        assert err <= 2.0 ** -7 * scale, f"max difference from the plain attention {err:.3e} on scale {scale:.3e}"


def test_the_largest_accepted_call_leaves_the_counters_usable():
    """A call whose partial results end just below the counters at the array's end, then a small call: had
    the first one written over the counters, or left one of them non-zero, the second would combine too
    early or never, and differ from the entry point that is given fresh counters."""
    fn, cap = bind()
    nh, hd, rows = 32, 64, 8
    most_splits = cap() // (rows * nh * (hd + 2))
    big = case(4, n_seq=rows, nh=nh, nkv=8, hd=hd, max_len=700, window=None)
    big = (*big[:6], int(most_splits), big[7])          # more splits than the sequences have: their blocks do nothing
    small = case(5, n_seq=2, nh=4, nkv=2, hd=128, max_len=500, window=200)
    for c in (big, small, big):
        out, ref = run_both(fn, c)
        assert torch.equal(out, ref)
    err = float((out.double().cpu() - plain_attention(big)).abs().max())
    assert err <= 2.0 ** -7 * float(plain_attention(big).abs().max())


def test_a_request_beyond_the_built_in_scratch_is_refused():
    fn, cap = bind()
    q, k, v, seq, pos, table, n_splits, (nh, nkv, hd, window) = case(3, n_seq=2, nh=4, nkv=4, hd=64, max_len=100, window=None)
    out = torch.zeros(2, nh * hd, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    big_splits = cap() // (2 * nh * (hd + 2)) + 1
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), seq.data_ptr(), pos.data_ptr(), table.data_ptr(),
            table.shape[1], k.shape[0], 64, 2, nh, nkv, hd, 0, SPLIT, int(big_splits), status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == TOO_LARGE
    assert torch.all(out == 0), "a refused call must not launch anything"
