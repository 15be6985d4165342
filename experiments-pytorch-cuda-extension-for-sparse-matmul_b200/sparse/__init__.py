"""Block-sparse attention primitives for NVIDIA B200 (sm_100a).

Same public surface as the reference package (sparse/__init__.py:1-2):
``SparseLayout`` and ``matmul``; ``softmax`` is the op the reference left
unbound (sparse_softmax.cu:208-236); ``attention`` fuses the three steps of
block-sparse attention into one kernel.
"""
from .layout import SparseLayout
from .matmul import matmul, SparseMatMul
from .softmax import softmax, SparseSoftmax
from .attention import attention, SparseAttention
from .module import BlockSparseSelfAttention
from .batched import BatchedSparseLayout, batched_matmul, batched_softmax, batched_attention

__all__ = ["SparseLayout", "matmul", "SparseMatMul", "softmax", "SparseSoftmax", "attention", "SparseAttention", "BlockSparseSelfAttention",
           "BatchedSparseLayout", "batched_matmul", "batched_softmax", "batched_attention"]
