"""Matrix products of the layers: ``out = a @ w.T``.

Which kernel runs is decided here and nowhere else:
* 32-bit engine, or a weight kept in 32-bit: the plain CUDA-core kernel with
  true float32 multiply-adds and a fixed summation order;
* bfloat16 activations and weights, at most SKINNY_ROWS rows (decode): the
  weight-streaming tensor-core kernel of this library;
* bfloat16 with more rows (prefill): a library product (cuBLAS through torch)
  with float32 accumulation and output, as the reference engine leaves its
  dense products to its tensor library.
"""
from __future__ import annotations

import torch

from ..csrc import ops

SKINNY_ROWS = 16            # dense products with at most this many rows stream the weights once
SKINNY_GROUPED_PAIRS = 1 << 30


def _both_bf16(a, w) -> bool:
    return a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16


def linear(rt, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """a [M,K] (activation dtype), w [N,K], out [M,N] float32."""
    if _both_bf16(a, w):
        if a.shape[0] <= SKINNY_ROWS and ops.skinny_fits(a.shape[1]):
            ops.gemm_skinny(a, w, out)
        else:
            torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
    else:
        ops.gemm_simt(a, w, out)
    return out


def swiglu_linear(rt, a, w_gate_up, act, tag):
    """act = silu(a @ w_gate.T) * (a @ w_up.T) in the activation dtype; w_gate_up
    is [2I, K] with the gate rows first."""
    n = a.shape[0]
    inter = w_gate_up.shape[0] // 2
    if _both_bf16(a, w_gate_up) and n <= SKINNY_ROWS and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w_gate_up, act, swiglu=True)
        return act
    gu = rt.ws.get(tag + "_gu", (n, 2 * inter), torch.float32)
    linear(rt, a, w_gate_up, gu)
    ops.swiglu(gu, act)
    return act


def grouped_swiglu_linear(rt, a, w_gate_up, act, group_offsets, a_rows, rows, max_rows, tag):
    """Grouped form of swiglu_linear: permuted row r reads a[a_rows[r]] and the
    weights of the group whose range holds r (w_gate_up [G, 2I, K])."""
    if _both_bf16(a, w_gate_up) and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w_gate_up, act, swiglu=True, a_rows=a_rows, group_offsets=group_offsets, rows=rows,
                        max_rows=max_rows)
        return act
    inter = w_gate_up.shape[1] // 2
    gu = rt.ws.get(tag + "_gu", (rows, 2 * inter), torch.float32)
    ops.gemm_simt(a, w_gate_up, gu, a_rows=a_rows, group_offsets=group_offsets, rows=rows)
    ops.swiglu(gu, act)
    return act


def grouped_linear(rt, a, w, out, group_offsets, row_scale, rows, max_rows):
    """out[r] = row_scale[r] * a[r] @ w[g].T for the rows of every group (w [G,N,K])."""
    if _both_bf16(a, w) and ops.skinny_fits(a.shape[1]):
        ops.gemm_skinny(a, w, out, row_scale=row_scale, group_offsets=group_offsets, rows=rows, max_rows=max_rows)
    else:
        ops.gemm_simt(a, w, out, row_scale=row_scale, group_offsets=group_offsets, rows=rows)
    return out
