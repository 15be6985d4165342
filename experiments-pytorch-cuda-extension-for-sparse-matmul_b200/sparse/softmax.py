"""Autograd op for the block-sparse row softmax.

The reference has the two C++ functions ``sparse_softmax_forward(x, row_blocks,
row_table)`` and ``sparse_softmax_backward(y, dy, row_blocks, row_table)``
(sparse_softmax.cu:208-236) but never binds them.  This op wires them to
autograd and adds a fused scale, a causal mask and a key-padding mask:

    y = softmax(scale * x + mask)   over each dense row, restricted to the layout

``x`` is ``[..., nnz, block, block]``.  ``causal`` masks key position > query
position (absolute positions, so it acts inside diagonal blocks).
``key_padding_mask`` is ``[batch, seq_k]`` with nonzero = padding; ``batch``
must divide the flattened leading dims of ``x`` (heads of one batch entry are
contiguous).  Rows with no unmasked element return zeros.
"""
from typing import Any, Optional, Tuple

import torch

from . import kernel
from .layout import SparseLayout


class SparseSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, layout: SparseLayout, scale: float = 1.0, causal: bool = False,
                key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        row_blocks, row_table = layout.row_layout
        if key_padding_mask is not None:
            # the kernels index the mask by absolute key position: it has to cover every block column
            keys = layout.pattern.size(1) * layout.block
            if key_padding_mask.dim() != 2 or key_padding_mask.size(1) < keys:
                raise ValueError("key_padding_mask must be [batch, seq_k] with seq_k >= %d, got shape %s"
                                 % (keys, tuple(key_padding_mask.shape)))
        y = kernel.sparse_ops.sparse_softmax_forward(x, row_blocks, row_table, float(scale), bool(causal),
                                                     key_padding_mask, getattr(layout, "max_row_blocks", 0))
        ctx.save_for_backward(y)
        ctx.layout, ctx.scale = layout, float(scale)
        return kernel.check(y)

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        (y,) = ctx.saved_tensors
        row_blocks, row_table = ctx.layout.row_layout
        dx = None
        if ctx.needs_input_grad[0]:
            dx = kernel.sparse_ops.sparse_softmax_backward(y, dy.contiguous(), row_blocks, row_table, ctx.scale,
                                                           getattr(ctx.layout, "max_row_blocks", 0))
        return kernel.check(dx), None, None, None, None


def softmax(x: torch.Tensor, layout: SparseLayout, scale: float = 1.0, causal: bool = False,
            key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    return SparseSoftmax.apply(x, layout, scale, causal, key_padding_mask)
