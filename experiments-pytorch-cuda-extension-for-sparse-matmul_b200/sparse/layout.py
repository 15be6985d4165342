"""Block layout of a block-sparse matrix.

Mirror of the reference ``SparseLayout`` (sparse/layout.py:5-57): same
constructor argument, attributes (``pattern``, ``sparse_positions``,
``row_layout``, ``col_layout``) and methods (``to_sparse``, ``to_dense``).
Differences, all additive:

* the descriptor tensors are built on the GPU by ``sparse_ops.build_layout``
  (bit-identical to the reference's host-side ``_create_layout``, :14-38);
* ``block`` is an attribute (16, 32, 64 or 128; the reference hard-codes 32);
* a ``bool`` pattern is accepted (the reference's ``index_add`` saturates on
  bool and yields a wrong offset table);
* ``to_dense`` zero-fills outside the layout (the reference leaves that
  memory uninitialised, :48) and both converters run as one kernel for CUDA
  tensors instead of a Python loop over the blocks.
"""
from typing import Tuple

import torch

from .kernel import sparse_ops


class SparseLayout:
    def __init__(self, pattern: torch.Tensor, block: int = 32, device=None):
        if pattern.dim() != 2:
            raise ValueError("pattern must be a 2-D tensor of 0/1 block flags, got shape %s"
                             % (tuple(pattern.shape),))
        if block not in (16, 32, 64, 128):
            raise ValueError("block must be 16, 32, 64 or 128, got %r" % (block,))
        if pattern.size(0) > 65535 or pattern.size(1) > 65535:
            raise ValueError("at most 65535 block rows / columns are supported")
        self.pattern = pattern
        self.block = block
        self.sparse_positions = torch.nonzero(pattern, as_tuple=False)

        if device is None:
            device = pattern.device if pattern.is_cuda else torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.row_layout, self.col_layout = self._create_layouts(pattern)
        # longest block row / column: a hint that lets the softmax cover every row in one launch
        on = pattern != 0
        self.max_row_blocks = int(on.sum(dim=1).max()) if on.numel() else 0
        self.max_col_blocks = int(on.sum(dim=0).max()) if on.numel() else 0

    def _create_layouts(self, pattern: torch.Tensor
                        ) -> Tuple[Tuple[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]:
        row_blocks, row_table, col_blocks, col_table = sparse_ops.build_layout(pattern.to(self.device))
        return (row_blocks, row_table), (col_blocks, col_table)

    @property
    def num_blocks(self) -> int:
        return self.row_layout[0].numel() // 2

    @property
    def shape(self) -> Tuple[int, int]:
        """Dense shape covered by the layout."""
        return self.pattern.size(0) * self.block, self.pattern.size(1) * self.block

    def to_sparse(self, x: torch.Tensor) -> torch.Tensor:
        """Gather the layout's blocks of a dense ``[..., R*block, C*block]`` tensor into
        ``[..., nnz, block, block]`` (reference sparse/layout.py:40-45)."""
        if x.is_cuda:
            return sparse_ops.dense_to_sparse(x, self.row_layout[0].to(x.device), self.pattern.size(0),
                                              self.pattern.size(1), self.block)
        b = self.block
        rows, cols = self.sparse_positions[:, 0], self.sparse_positions[:, 1]
        tiles = x.reshape(x.shape[:-2] + (self.pattern.size(0), b, self.pattern.size(1), b))
        return tiles[..., rows, :, cols, :].movedim(0, -3) if rows.numel() else \
            x.new_zeros(x.shape[:-2] + (0, b, b))

    def to_dense(self, x: torch.Tensor) -> torch.Tensor:
        """Scatter ``[..., nnz, block, block]`` back into a dense tensor, zero outside the
        layout (reference sparse/layout.py:47-57)."""
        if x.is_cuda:
            return sparse_ops.sparse_to_dense(x, self.row_layout[0].to(x.device), self.pattern.size(0),
                                              self.pattern.size(1), self.block)
        b = self.block
        out = x.new_zeros(x.shape[:-3] + (self.pattern.size(0) * b, self.pattern.size(1) * b))
        for k, (i, j) in enumerate(self.sparse_positions.tolist()):
            out[..., i * b:(i + 1) * b, j * b:(j + 1) * b] = x[..., k, :, :]
        return out
