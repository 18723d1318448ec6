"""Matrix products of the layers: ``out = a @ w.T`` with float32 output.

Which kernel runs is decided here and nowhere else:
* 32-bit engine, or a weight kept in 32-bit: the plain CUDA-core kernel with
  true float32 multiply-adds and a fixed summation order;
* bfloat16 activations and weights: a library product (cuBLAS through torch)
  with float32 accumulation and output, as the reference engine leaves its
  dense products to its tensor library.
"""
from __future__ import annotations

import torch

from ..csrc import ops


def linear(rt, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """a [M,K] (activation dtype), w [N,K], out [M,N] float32."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
    else:
        ops.gemm_simt(a, w, out)
    return out


def grouped_linear(rt, a, w, out, group_offsets, a_rows=None, row_scale=None, rows=None):
    """Rows sorted by group; group g multiplies its rows with w[g] ([G,N,K])."""
    ops.gemm_simt(a, w, out, a_rows=a_rows, row_scale=row_scale, group_offsets=group_offsets, rows=rows)
    return out
