"""Fused block-sparse attention.

    out = softmax(scale * Q K^T + masks, restricted to the layout) V

The reference has no such op: a caller composes it from its matmul in "sdd"
mode (sparse/matmul.py:55-57), a softmax and its matmul in "dsd" mode, and
every step writes the ``[..., nnz, block, block]`` tensor to memory.
``attention`` computes the same result in one kernel launch where the fused
kernel applies (fp16 / bf16, block 32, 64 or 128, head dim 64 or 128) and
composes the three unfused ops otherwise, so it can be called for any layout
and dtype.  The kernels work on 64 x 64 blocks and touch no sparse tensor,
only the positions of the blocks: a block-128 layout runs as the block-64
layout with every block split in 2 x 2, a block-32 layout (with an even
number of block rows and columns) as the layout of the 64 x 64 blocks that
contain its blocks, each with a 4-bit mask of the 32 x 32 quadrants that
belong to the layout (carried in the descriptors' idx field, which the fused
kernels do not use); the element-level masks do not depend on the block size.

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
    rows, cols = layout.pattern.size(0), layout.pattern.size(1)
    if layout.block == 32:
        shape_ok = rows % 2 == 0 and cols % 2 == 0
    elif layout.block == 128:
        shape_ok = 2 * rows <= 65535 and 2 * cols <= 65535
    else:
        shape_ok = layout.block == 64
    return q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and shape_ok and q.size(-1) in (64, 128)


class _KernelLayout:
    """What the fused kernels get: row / column descriptors of 64 x 64 blocks and the quadrant flag."""

    def __init__(self, row_layout, col_layout, block_cols: int, quadrant_masks: bool):
        self.row_layout, self.col_layout = row_layout, col_layout
        self.block_cols, self.quadrant_masks = block_cols, quadrant_masks


def _kernel_layout(layout: SparseLayout) -> _KernelLayout:
    """The layout in the kernels' 64 x 64 blocks (built once per layout object)."""
    cached = getattr(layout, "_fused_layout", None)
    if cached is not None:
        return cached
    if layout.block == 64:
        fine = _KernelLayout(layout.row_layout, layout.col_layout, layout.pattern.size(1), False)
    elif layout.block == 128:
        pattern = (layout.pattern != 0).to(torch.uint8).repeat_interleave(2, 0).repeat_interleave(2, 1)
        split = SparseLayout(pattern, block=64, device=layout.device)
        fine = _KernelLayout(split.row_layout, split.col_layout, pattern.size(1), False)
    else:
        on = (layout.pattern != 0).to(torch.int32).cpu()
        rows, cols = on.size(0) // 2, on.size(1) // 2
        quads = on.reshape(rows, 2, cols, 2)
        # bit 2 * row_half + col_half of a coarse block = its 32 x 32 quadrant is in the layout
        bits = quads[:, 0, :, 0] + 2 * quads[:, 0, :, 1] + 4 * quads[:, 1, :, 0] + 8 * quads[:, 1, :, 1]
        coarse = SparseLayout((bits != 0).to(torch.uint8), block=64, device=layout.device)
        rank_bits = bits[bits != 0].to(device=layout.device, dtype=torch.int32)      # by row-major rank

        def with_masks(blocks: torch.Tensor) -> torch.Tensor:
            pairs = blocks.view(-1, 2).clone()
            pairs[:, 0] = rank_bits[pairs[:, 0].long()]        # idx (the rank) -> the block's quadrant mask
            return pairs.view(-1).contiguous()

        fine = _KernelLayout((with_masks(coarse.row_layout[0]), coarse.row_layout[1]),
                             (with_masks(coarse.col_layout[0]), coarse.col_layout[1]), cols, True)
    layout._fused_layout = fine
    return fine


def _fused_forward(q, k, v, layout, scale, causal, key_padding_mask):
    fine = _kernel_layout(layout)
    return kernel.sparse_ops.sparse_attention_forward(
        q, k, v, fine.row_layout[0], fine.row_layout[1], 64, fine.block_cols, float(scale), bool(causal),
        key_padding_mask, fine.quadrant_masks)


class SparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: SparseLayout,
                scale: float = 1.0, causal: bool = False,
                key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        out, lse = _fused_forward(q, k, v, layout, scale, causal, key_padding_mask)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.layout, ctx.scale, ctx.causal, ctx.kpm = layout, float(scale), bool(causal), key_padding_mask
        return kernel.check(out)

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        q, k, v, out, lse = ctx.saved_tensors
        layout, ops = ctx.layout, kernel.sparse_ops
        if fused_backward:
            fine = _kernel_layout(layout)
            dq, dk, dv = ops.sparse_attention_backward(
                q, k, v, out, dout.contiguous(), lse, fine.row_layout[0], fine.row_layout[1],
                fine.col_layout[0], fine.col_layout[1], 64, ctx.scale, ctx.causal, ctx.kpm, fine.quadrant_masks)
            kernel.check(dout)
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
        kernel.check(dout)
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
