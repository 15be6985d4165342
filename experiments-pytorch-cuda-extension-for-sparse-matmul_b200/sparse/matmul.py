"""Autograd op for the block-sparse matmul.

Same contract as the reference ``SparseMatMul`` (sparse/matmul.py:7-57):
``matmul(a, b, mode, layout, trans_a=False, trans_b=False)`` where the three
letters of ``mode`` give the sparsity of (output, a, b).  The backward pass
derives both gradients by permuting the mode letters and the transposition
flags exactly as the reference does (:30-50); all twelve
(mode, trans_a, trans_b) products it can request are implemented by the
native library.
"""
from typing import Any, Optional, Tuple

import torch

from . import kernel
from .layout import SparseLayout


def _ops():
    return kernel.sparse_ops


class SparseMatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, a: torch.Tensor, b: torch.Tensor, mode: str, layout: SparseLayout,
                trans_a: bool = False, trans_b: bool = False) -> torch.Tensor:
        if mode not in ("sdd", "dsd", "dds"):
            raise ValueError("mode must be 'sdd', 'dsd' or 'dds', got %r" % (mode,))
        ctx.save_for_backward(a, b)
        ctx.mode, ctx.layout = mode, layout
        ctx.trans_a, ctx.trans_b = bool(trans_a), bool(trans_b)
        return kernel.check(_ops().sparse_matmul(a, b, mode, layout.row_layout, layout.col_layout,
                                                 ctx.trans_a, ctx.trans_b, layout.block))

    @staticmethod
    def backward(ctx: Any, dc: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        da, db, dc = None, None, dc.contiguous()
        a, b = ctx.saved_tensors
        mode, layout = ctx.mode, ctx.layout
        trans_a, trans_b = ctx.trans_a, ctx.trans_b
        out_s, a_s, b_s = mode[0], mode[1], mode[2]

        if ctx.needs_input_grad[0]:
            # dA = dC . op(B)^T, or its transpose when A itself is transposed.
            da_mode = (a_s + b_s + out_s) if trans_a else (a_s + out_s + b_s)
            lhs, rhs = (b, dc) if trans_a else (dc, b)
            da = _ops().sparse_matmul(lhs, rhs, da_mode, layout.row_layout, layout.col_layout,
                                      trans_a and trans_b, trans_a or not trans_b, layout.block)
        if ctx.needs_input_grad[1]:
            # dB = op(A)^T . dC, or its transpose when B itself is transposed.
            db_mode = (b_s + out_s + a_s) if trans_b else (b_s + a_s + out_s)
            lhs, rhs = (dc, a) if trans_b else (a, dc)
            db = _ops().sparse_matmul(lhs, rhs, db_mode, layout.row_layout, layout.col_layout,
                                      not trans_a or trans_b, trans_a and trans_b, layout.block)
        kernel.check(dc)
        return da, db, None, None, None, None


# Call the op through this function, as in the reference (sparse/matmul.py:55-57).
matmul = SparseMatMul.apply
