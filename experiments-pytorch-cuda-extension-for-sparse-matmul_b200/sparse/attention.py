"""Fused block-sparse attention.

    out = softmax(scale * Q K^T + masks, restricted to the layout) V

The reference has no such op: a caller composes it from its matmul in "sdd"
mode (sparse/matmul.py:55-57), a softmax and its matmul in "dsd" mode, and
every step writes the ``[..., nnz, block, block]`` tensor to memory.
``attention`` computes the same result in one kernel launch where the fused
kernel applies (fp16 / bf16, block 64 or 128, head dim 64 or 128) and composes
the three unfused ops otherwise, so it can be called for any layout and dtype.
The kernel works on 64 x 64 blocks and touches no sparse tensor, only the
positions of the blocks: a block-128 layout runs as the block-64 layout with
every block split in 2 x 2 (the element-level masks do not depend on the
block size).

The backward pass of the fused path is fused as well: the forward keeps only
the output and the row log-sum-exp, and two kernels (dQ by block rows; dK and
dV by block columns) recompute the probabilities on chip:

    P  = exp(scale * Q K^T - lse)              dV = P^T dO
    dP = dO V^T                                dS = scale * P o (dP - rowsum(dO o O))
    dQ = dS K                                  dK = dS^T Q

``fused_backward = False`` selects the same gradients composed from the
unfused kernels (sdd, softmax, softmax backward, dsd).
"""
from typing import Any, Optional, Tuple

import torch

from . import kernel
from .layout import SparseLayout
from .matmul import matmul
from .softmax import softmax


fused_backward = True      # False: compose the backward of the fused forward from the unfused kernels


def fused_supported(q: torch.Tensor, layout: SparseLayout) -> bool:
    """True where the one-kernel forward applies."""
    return (q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and layout.block in (64, 128)
            and 2 * layout.pattern.size(0) <= 65535 and 2 * layout.pattern.size(1) <= 65535
            and q.size(-1) in (64, 128))


def _kernel_layout(layout: SparseLayout) -> SparseLayout:
    """The layout in the kernel's 64 x 64 blocks (built once per layout object)."""
    if layout.block == 64:
        return layout
    split = getattr(layout, "_split64", None)
    if split is None:
        pattern = (layout.pattern != 0).to(torch.uint8).repeat_interleave(2, 0).repeat_interleave(2, 1)
        split = SparseLayout(pattern, block=64, device=layout.device)
        layout._split64 = split
    return split


def _fused_forward(q, k, v, layout, scale, causal, key_padding_mask):
    fine = _kernel_layout(layout)
    row_blocks, row_table = fine.row_layout
    return kernel.sparse_ops.sparse_attention_forward(
        q, k, v, row_blocks, row_table, 64, fine.pattern.size(1), float(scale), bool(causal), key_padding_mask)


class SparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: SparseLayout,
                scale: float = 1.0, causal: bool = False,
                key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        out, lse = _fused_forward(q, k, v, layout, scale, causal, key_padding_mask)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.layout, ctx.scale, ctx.causal, ctx.kpm = layout, float(scale), bool(causal), key_padding_mask
        return out

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        q, k, v, out, lse = ctx.saved_tensors
        layout, ops = ctx.layout, kernel.sparse_ops
        if fused_backward:
            fine = _kernel_layout(layout)
            dq, dk, dv = ops.sparse_attention_backward(
                q, k, v, out, dout.contiguous(), lse, fine.row_layout[0], fine.row_layout[1],
                fine.col_layout[0], fine.col_layout[1], 64, ctx.scale, ctx.causal, ctx.kpm)
            return dq, dk, dv, None, None, None, None
        rows, cols, block = layout.row_layout, layout.col_layout, layout.block
        hint = getattr(layout, "max_row_blocks", 0)
        dout = dout.contiguous()
        s = ops.sparse_matmul(q, k, "sdd", rows, cols, False, True, block)
        p = ops.sparse_softmax_forward(s, rows[0], rows[1], ctx.scale, ctx.causal, ctx.kpm, hint)
        dq = dk = dv = None
        if ctx.needs_input_grad[2]:
            dv = ops.sparse_matmul(p, dout, "dsd", rows, cols, True, False, block)
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            dp = ops.sparse_matmul(dout, v, "sdd", rows, cols, False, True, block)
            ds = ops.sparse_softmax_backward(p, dp, rows[0], rows[1], ctx.scale, hint)
            if ctx.needs_input_grad[0]:
                dq = ops.sparse_matmul(ds, k, "dsd", rows, cols, False, False, block)
            if ctx.needs_input_grad[1]:
                dk = ops.sparse_matmul(ds, q, "dsd", rows, cols, True, False, block)
        return dq, dk, dv, None, None, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: SparseLayout, scale: float = 1.0,
              causal: bool = False, key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-sparse attention of ``q [..., seq_q, d]`` over ``k, v [..., seq_k, d]``."""
    if fused_supported(q, layout):
        return SparseAttention.apply(q, k, v, layout, scale, causal, key_padding_mask)
    scores = matmul(q, k, "sdd", layout, False, True)
    probs = softmax(scores, layout, scale, causal, key_padding_mask)
    return matmul(probs, v, "dsd", layout, False, False)


def attention_lse(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: SparseLayout, scale: float = 1.0,
                  causal: bool = False, key_padding_mask: Optional[torch.Tensor] = None):
    """Forward only: (output, log-sum-exp of the scaled masked scores per query row)."""
    return _fused_forward(q, k, v, layout, scale, causal, key_padding_mask)
