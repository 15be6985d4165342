"""One layout per head, one kernel launch for all heads.

The reference ``SparseLayout`` takes a single 2-D pattern (sparse/layout.py:6-12;
``pattern.t()`` at :17 rules out a batch of patterns), so a model whose heads
use different patterns needs one layout object and one launch per head.
``BatchedSparseLayout`` keeps the kernels and the wire format unchanged and
moves the heads into the block grid instead: the ``H`` patterns ``[R, C]``
become the diagonal blocks of one ``[H*R, H*C]`` super-pattern, and a dense
operand ``[..., H, seq, d]`` is read as ``[..., H*seq, d]`` -- the same memory,
since the heads of one batch entry are contiguous.  Block row ``h*R + r`` of the
super-layout then is block row ``r`` of head ``h``, and its blocks point at
block columns ``h*C + c``, i.e. at rows of head ``h`` in the folded key / value
operand.  Every kernel (both matmul engines, the softmax, the fused attention)
runs on the super-layout as it is; the causal mask compares positions that
carry the same per-head offset, so it is unchanged for square patterns.

Sparse tensors are ``[..., nnz_total, block, block]`` with the blocks of head 0
first (``head_slices`` gives each head's range), dense tensors
``[..., H, seq, d]``.
"""
from typing import List, Optional

import torch

from .attention import attention
from .layout import SparseLayout
from .matmul import matmul
from .softmax import softmax


class BatchedSparseLayout:
    def __init__(self, patterns: torch.Tensor, block: int = 32, device=None):
        if patterns.dim() != 3:
            raise ValueError("patterns must be [heads, block_rows, block_cols], got shape %s" % (tuple(patterns.shape),))
        heads, rows, cols = patterns.shape
        if heads * rows > 65535 or heads * cols > 65535:
            raise ValueError("heads * block rows (columns) must not exceed 65535")
        self.patterns = patterns
        self.heads, self.rows, self.cols, self.block = heads, rows, cols, block
        on = (patterns != 0).to(torch.uint8).cpu()
        super_pattern = torch.zeros(heads * rows, heads * cols, dtype=torch.uint8)
        for h in range(heads):
            super_pattern[h * rows:(h + 1) * rows, h * cols:(h + 1) * cols] = on[h]
        self.layout = SparseLayout(super_pattern, block=block, device=device)
        counts = on.flatten(1).sum(dim=1).tolist()
        self.head_slices: List[slice] = []
        start = 0
        for n in counts:
            self.head_slices.append(slice(start, start + int(n)))
            start += int(n)

    @property
    def num_blocks(self) -> int:
        return self.layout.num_blocks

    def fold(self, x: torch.Tensor) -> torch.Tensor:
        """``[..., H, seq, d]`` -> ``[..., H * seq, d]`` (a view for contiguous input)."""
        if x.dim() < 3 or x.size(-3) != self.heads:
            raise ValueError("expected [..., %d, seq, d], got shape %s" % (self.heads, tuple(x.shape)))
        return x.reshape(x.shape[:-3] + (self.heads * x.size(-2), x.size(-1)))

    def unfold(self, x: torch.Tensor) -> torch.Tensor:
        """``[..., H * seq, d]`` -> ``[..., H, seq, d]``."""
        return x.reshape(x.shape[:-2] + (self.heads, x.size(-2) // self.heads, x.size(-1)))

    def head_blocks(self, x: torch.Tensor, head: int) -> torch.Tensor:
        """The blocks of one head inside a sparse ``[..., nnz_total, block, block]`` tensor."""
        return x[..., self.head_slices[head], :, :]


def batched_matmul(a: torch.Tensor, b: torch.Tensor, mode: str, layout: BatchedSparseLayout,
                   trans_a: bool = False, trans_b: bool = False) -> torch.Tensor:
    """``sparse.matmul`` with one pattern per head.  Dense operands and results are
    ``[..., H, seq, d]``: the sequence must be the row dimension in memory (sdd: ``a`` plain, ``b``
    with ``trans_b``; dsd: ``b`` plain; dds: ``a`` with ``trans_a``), which is what attention uses."""
    if mode not in ("sdd", "dsd", "dds"):
        raise ValueError("mode must be 'sdd', 'dsd' or 'dds', got %r" % (mode,))
    if mode == "sdd":
        if trans_a or not trans_b:
            raise ValueError("batched sdd needs a [..., H, seq_q, d] and b [..., H, seq_k, d] with trans_b=True")
        return matmul(layout.fold(a), layout.fold(b), "sdd", layout.layout, False, True)
    if mode == "dsd":
        if trans_b:
            raise ValueError("batched dsd needs b as [..., H, seq, d] (trans_b=False)")
        return layout.unfold(matmul(a, layout.fold(b), "dsd", layout.layout, trans_a, False))
    if not trans_a:
        raise ValueError("batched dds needs a as [..., H, seq, d] with trans_a=True")
    out = matmul(layout.fold(a), b, "dds", layout.layout, True, trans_b)      # [..., d, H * seq]
    return out.reshape(out.shape[:-1] + (layout.heads, out.size(-1) // layout.heads)).transpose(-3, -2)


def batched_softmax(x: torch.Tensor, layout: BatchedSparseLayout, scale: float = 1.0, causal: bool = False,
                    key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sparse.softmax`` with one pattern per head (``key_padding_mask`` is ``[batch, seq_k]`` as usual)."""
    if key_padding_mask is not None:
        key_padding_mask = key_padding_mask.repeat(1, layout.heads)      # key positions carry the head offset
    if causal and layout.rows != layout.cols:
        raise ValueError("the causal mask needs square per-head patterns")
    return softmax(x, layout.layout, scale, causal, key_padding_mask)


def batched_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: BatchedSparseLayout,
                      scale: float = 1.0, causal: bool = False,
                      key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sparse.attention`` with one pattern per head: q, k, v and the result are ``[..., H, seq, d]``."""
    if key_padding_mask is not None:
        key_padding_mask = key_padding_mask.repeat(1, layout.heads)
    if causal and layout.rows != layout.cols:
        raise ValueError("the causal mask needs square per-head patterns")
    out = attention(layout.fold(q), layout.fold(k), layout.fold(v), layout.layout, scale, causal, key_padding_mask)
    return layout.unfold(out)
