"""Multi-head block-sparse self-attention as an ``nn.Module``.

The reference stops at the operators (sparse/__init__.py:1-2 exports a layout
class and a matmul); this is the caller a user of those operators writes on
top of them: packed QKV projection, ``attention`` over a ``SparseLayout``,
output projection.  Blocks 32 (even block grid), 64 and 128 with head dimension
64 or 128 in fp16 / bf16 run the fused forward and backward kernels; every
other combination composes the unfused operators.
"""
from typing import Optional

import torch
from torch import nn

from .attention import attention
from .layout import SparseLayout


class BlockSparseSelfAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, layout: SparseLayout, causal: bool = False,
                 bias: bool = True, device=None, dtype=None):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be a multiple of num_heads")
        if layout.pattern.size(0) != layout.pattern.size(1):
            raise ValueError("self-attention needs a square block pattern")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.layout, self.causal = layout, causal
        self.scale = self.head_dim ** -0.5
        self.qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=bias, device=device, dtype=dtype)
        self.out = nn.Linear(embed_dim, embed_dim, bias=bias, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor, key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x``: [batch, seq, embed_dim] with seq = block rows * block; ``key_padding_mask``:
        [batch, seq], nonzero = padding."""
        batch, seq, _ = x.shape
        if seq != self.layout.pattern.size(0) * self.layout.block:
            raise ValueError("sequence length %d does not match the layout (%d)" %
                             (seq, self.layout.pattern.size(0) * self.layout.block))
        qkv = self.qkv(x).view(batch, seq, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        q, k, v = (t.contiguous() for t in qkv)                       # [batch, heads, seq, head_dim]
        ctx = attention(q, k, v, self.layout, self.scale, self.causal, key_padding_mask)
        return self.out(ctx.transpose(1, 2).reshape(batch, seq, self.embed_dim))
