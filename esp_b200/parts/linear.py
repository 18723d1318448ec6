"""Matrix products of the layers: ``out = a @ w.T``.

Which kernel runs is decided here and nowhere else:
* 32-bit engine, or a weight kept in 32-bit: the plain CUDA-core kernel with
  true float32 multiply-adds and a fixed summation order;
* bfloat16 activations and weights, at most SKINNY_ROWS rows (decode): the
  weight-streaming tensor-core kernel of this library (grouped products: see
  ``grouped_uses_tc05``);
* bfloat16 with more rows (prefill): a library product (cuBLAS through torch)
  with float32 accumulation and output, as the reference engine leaves its
  dense products to its tensor library.
"""
from __future__ import annotations

import torch

from ..csrc import ops

import os

# dense products with at most this many rows stream the weights once through the kernel's one block of eight
# rows (the kernel takes 16 in two blocks, which is slower than the library product from 9 rows on: batch 16 at
# the A2.7B sizes 6.75 against 6.37 ms a step)
SKINNY_ROWS = int(os.environ.get("ESP_B200_SKINNY_ROWS", "8"))
TC05_GROUPED_ROWS = int(os.environ.get("ESP_B200_TC05_ROWS", "128"))   # grouped products with at least this many (token, expert) rows use TMA + tcgen05
TC05_GROUP_ROWS = int(os.environ.get("ESP_B200_TC05_GROUP_ROWS", "8"))   # ... or with a group that may have more rows than this
# dense products with many rows: "own" = this library's TMA + tcgen05 kernel everywhere; "library" = cuBLAS
# through torch; "mixed" = cuBLAS for plain products, this library's kernel where SwiGLU is fused into it
DENSE_GEMM = os.environ.get("ESP_B200_DENSE_GEMM", "mixed")


def _both_bf16(a, w) -> bool:
    return a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16


def linear(rt, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """a [M,K] (activation dtype), w [N,K], out [M,N] float32."""
    if _both_bf16(a, w):
        if a.shape[0] <= SKINNY_ROWS and ops.skinny_fits(a.shape[1]):
            ops.gemm_skinny(a, w, out)
        elif DENSE_GEMM == "own" and a.shape[1] % 8 == 0 and a.is_contiguous() and out.is_contiguous():
            ops.gemm_tc05(a, w, out, rt.status)
        else:
            torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
    else:
        ops.gemm_simt(a, w, out)
    return out


def swiglu_linear(rt, a, w_gate_up, act, tag, max_ctas=0):
    """act = silu(a @ w_gate.T) * (a @ w_up.T) in the activation dtype; w_gate_up
    is [2I, K] with the gate rows first.  ``max_ctas`` > 0 bounds the SMs that the
    many-row kernel takes."""
    n = a.shape[0]
    inter = w_gate_up.shape[0] // 2
    if _both_bf16(a, w_gate_up) and n <= SKINNY_ROWS and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w_gate_up, act, swiglu=True)
        return act
    if _both_bf16(a, w_gate_up) and DENSE_GEMM in ("own", "mixed") and a.shape[1] % 8 == 0 and a.is_contiguous() and act.is_contiguous():
        ops.gemm_tc05(a, w_gate_up, act, rt.status, swiglu=True, max_ctas=max_ctas)
        return act
    gu = rt.ws.get(tag + "_gu", (n, 2 * inter), torch.float32)
    linear(rt, a, w_gate_up, gu)
    ops.swiglu(gu, act)
    return act


def grouped_uses_tc05(a, w, rows, max_rows=None) -> bool:
    """Whether a grouped product of ``rows`` (token, expert) rows, at most ``max_rows`` of them in one group,
    runs on TMA + tcgen05.  The weight-streaming kernel keeps a group's rows in one or two blocks of eight; with
    one block it wins up to about 32 rows in all, with two it loses from the start (24 layers at the A2.7B
    sizes, context 4,096: batch 8 4.13 against 4.86 ms a step, batch 10 6.08 against 5.66, batch 16 7.42 against
    6.75, batch 64 14.9 against 13.5)."""
    many = rows >= TC05_GROUPED_ROWS or (max_rows is not None and max_rows > TC05_GROUP_ROWS)
    return _both_bf16(a, w) and many and a.shape[1] % 8 == 0 and w.shape[1] % 16 == 0


def grouped_swiglu_linear(rt, a, w_gate_up, act, group_offsets, a_rows, rows, max_rows, tag, tiles=None):
    """Grouped form of swiglu_linear: permuted row r reads a[a_rows[r]] and the
    weights of the group whose range holds r (w_gate_up [G, 2I, K]).  With
    ``tiles`` (the row-tile list of the permutation) the rows are gathered
    once and the product runs on TMA + tcgen05."""
    if tiles is not None:
        gathered = rt.ws.get(tag + "_gathered", (rows, a.shape[1]), torch.bfloat16)
        ops.gather_rows(a, a_rows, gathered)
        ops.gemm_tc05(gathered, w_gate_up, act, rt.status, swiglu=True, tiles=tiles)
        return act
    if _both_bf16(a, w_gate_up) and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w_gate_up, act, swiglu=True, a_rows=a_rows, group_offsets=group_offsets, rows=rows,
                        max_rows=max_rows)
        return act
    inter = w_gate_up.shape[1] // 2
    gu = rt.ws.get(tag + "_gu", (rows, 2 * inter), torch.float32)
    ops.gemm_simt(a, w_gate_up, gu, a_rows=a_rows, group_offsets=group_offsets, rows=rows)
    ops.swiglu(gu, act)
    return act


def grouped_linear(rt, a, w, out, group_offsets, row_scale, rows, max_rows, tiles=None, offsets_ready=False):
    """out[r] = row_scale[r] * a[r] @ w[g].T for the rows of every group (w [G,N,K]).  ``offsets_ready``: the
    kernel that ran right before this call did not write ``group_offsets`` or ``row_scale`` (it made ``a``)."""
    if tiles is not None:
        ops.gemm_tc05(a, w, out, rt.status, row_scale=row_scale, tiles=tiles)
        return out
    if _both_bf16(a, w) and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w, out, row_scale=row_scale, group_offsets=group_offsets, rows=rows, max_rows=max_rows,
                        offsets_ready=offsets_ready)
    else:
        ops.gemm_simt(a, w, out, row_scale=row_scale, group_offsets=group_offsets, rows=rows)
    return out
