"""CPU oracle for the block-sparse attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this file: only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` use it, as the checker and as the timed CPU baseline.

What it restates (file:line relative to the reference project root):

* ``create_layout`` -- ``SparseLayout._create_layout`` (sparse/layout.py:14-38),
  restated with numpy integer arithmetic.  PINNED: ``tests/golden/layout_*.json``
  were produced by executing the reference's own ``sparse/layout.py`` on the
  CPU (``tests/golden/make_golden.py``) and this restatement reproduces them
  bit for bit.
* ``sparse_matmul`` -- the semantics of ``sparse_matmul``
  (sparse/native/sparse_kernels.cc:7-50) as the autograd layer
  (sparse/matmul.py:30-50) requires them: ``op(A) @ op(B)`` computed densely in
  fp32/fp64 with the sparse operand zero outside the layout, and the output
  gathered into blocks for ``sdd``.  The reference has no tests or golden
  vectors for this and its CUDA kernels are wrong for 5 of the 12
  (mode, trans_a, trans_b) variants (dsd with trans_a, dds with trans_b,
  sdd with trans_a only), so the definition is pinned by the property the
  reference's own backward relies on: run through the reference's unmodified
  ``sparse/matmul.py`` this function yields gradients equal to dense autograd
  for all 12 variants (``tests/golden/autograd_table.json`` records the calls
  the reference's backward makes; ``tests/test_oracle.py`` checks both).
* ``softmax_forward`` / ``softmax_backward`` -- the math of
  ``sparse_softmax_32x32_{forward,backward}_kernel`` (sparse_softmax.cu:113-205):
  softmax over the elements of each dense row that lie in nonzero blocks.
  The reference file does not compile (undefined macros) and has no vectors, so
  no reference OUTPUT exists to compare with; the definition (masked dense torch
  softmax) is pinned to the reference SOURCE instead:
  ``reference_softmax_forward_emulated`` / ``..._backward_emulated`` replay the
  two kernels' arithmetic literally on the CPU (the ``-1e5f`` seed of the row
  maximum, :24; the strided walk of the row's blocks by 32 x 32 threads and the
  shuffle / shared-memory reduction trees, :26-55 and :75-104;
  ``__expf(x - max)`` then division by the row sum, :139-154;
  ``dx = (dy - sum(dy * y)) * y``, :190-203), and ``tests/test_oracle.py``
  checks that the definition equals that replay (scale 1, no masks) -- and
  documents the one place they differ: a row whose maximum lies below -1e5.
  Scale, causal and key-padding masks are additions of this build.
* ``strided_local_pattern`` -- the benchmark workload's block pattern, so that
  the CPU arm of ``bench.py`` needs nothing from the shipped package.
"""
from typing import Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------- layout
def create_layout(pattern, transpose: bool = False) -> Tuple[np.ndarray, np.ndarray]:
    """(blocks int32[2*nnz], offset_table int32[groups+1]) of a 2-D 0/1 pattern.

    Follows sparse/layout.py:14-38: nonzero positions in row-major order (or
    column-major for ``transpose``), idx = rank of the block in row-major
    nonzero order, packed_pos = (row << 16) + col, and an exclusive scan of the
    per-group block counts.
    """
    p = np.asarray(pattern.cpu() if isinstance(pattern, torch.Tensor) else pattern)
    if p.ndim != 2:
        raise ValueError("pattern must be 2-D")
    on = p != 0
    if transpose:
        cols, rows = np.nonzero(on.T)          # sorted by (col, row)
    else:
        rows, cols = np.nonzero(on)            # sorted by (row, col)
    rank = np.cumsum(on.reshape(-1).astype(np.int64)) - 1
    idx = rank[rows * p.shape[1] + cols]
    packed = (rows.astype(np.int64) << 16) + cols
    blocks = np.stack((idx, packed), axis=1).astype(np.int32).reshape(-1)
    keys = cols if transpose else rows
    groups = p.shape[1] if transpose else p.shape[0]
    counts = np.bincount(keys, minlength=groups)
    table = np.concatenate(([0], np.cumsum(counts))).astype(np.int32)
    return blocks, table


def sparse_positions(pattern) -> np.ndarray:
    """Row-major (row, col) list of the nonzero blocks (sparse/layout.py:8)."""
    p = np.asarray(pattern.cpu() if isinstance(pattern, torch.Tensor) else pattern)
    return np.stack(np.nonzero(p != 0), axis=1)


def to_sparse(x: torch.Tensor, pattern, block: int) -> torch.Tensor:
    """Gather blocks (sparse/layout.py:40-45 with 32 -> block)."""
    pos = sparse_positions(pattern)
    if len(pos) == 0:
        return x.new_zeros(x.shape[:-2] + (0, block, block))
    return torch.stack([x[..., i * block:(i + 1) * block, j * block:(j + 1) * block] for i, j in pos], dim=-3)


def to_dense(x: torch.Tensor, pattern, block: int) -> torch.Tensor:
    """Scatter blocks into a zero matrix (sparse/layout.py:47-57; zero fill instead of new_empty)."""
    p = np.asarray(pattern.cpu() if isinstance(pattern, torch.Tensor) else pattern)
    out = x.new_zeros(x.shape[:-3] + (p.shape[0] * block, p.shape[1] * block))
    for k, (i, j) in enumerate(sparse_positions(p)):
        out[..., i * block:(i + 1) * block, j * block:(j + 1) * block] = x[..., k, :, :]
    return out


def element_mask(pattern, block: int) -> torch.Tensor:
    """Boolean [R*block, C*block] mask of the elements covered by the layout."""
    p = torch.as_tensor(np.asarray(pattern.cpu() if isinstance(pattern, torch.Tensor) else pattern) != 0)
    return p.repeat_interleave(block, 0).repeat_interleave(block, 1)


# --------------------------------------------------------------------------- matmul
def sparse_matmul(a: torch.Tensor, b: torch.Tensor, mode: str, pattern, block: int,
                  trans_a: bool = False, trans_b: bool = False, dtype=torch.float32) -> torch.Tensor:
    """Masked dense definition of the block-sparse product (see module docstring).

    ``mode`` letters are the sparsity of (output, a, b).  Computation happens in
    ``dtype`` (fp32 by default, fp64 for tight checks) and the result is
    returned in that dtype.
    """
    if mode not in ("sdd", "dsd", "dds"):
        raise ValueError(mode)
    a = a.detach().cpu().to(dtype)
    b = b.detach().cpu().to(dtype)
    if mode[1] == "s":
        a = to_dense(a, pattern, block)
    if mode[2] == "s":
        b = to_dense(b, pattern, block)
    if trans_a:
        a = a.transpose(-1, -2)
    if trans_b:
        b = b.transpose(-1, -2)
    c = a @ b
    if mode[0] == "s":
        c = to_sparse(c, pattern, block)
    return c.contiguous()


# --------------------------------------------------------------------------- softmax
def _score_mask(pattern, block: int, causal: bool, key_padding_mask: Optional[torch.Tensor],
                batch_shape) -> torch.Tensor:
    """True where a score takes part in the softmax; broadcastable to [*batch, S_q, S_k]."""
    keep = element_mask(pattern, block)
    s_q, s_k = keep.shape
    if causal:
        q = torch.arange(s_q).unsqueeze(1)
        k = torch.arange(s_k).unsqueeze(0)
        keep = keep & (k <= q)
    keep = keep.expand(tuple(batch_shape) + keep.shape)
    if key_padding_mask is not None:
        kpm = key_padding_mask.cpu() != 0                      # [batch, s_k], True = padding
        z = int(np.prod(batch_shape)) if len(batch_shape) else 1
        per = z // kpm.shape[0]
        kpm = kpm.repeat_interleave(per, 0).reshape(tuple(batch_shape) + (1, s_k))
        keep = keep & ~kpm
    return keep


def softmax_forward(x: torch.Tensor, pattern, block: int, scale: float = 1.0, causal: bool = False,
                    key_padding_mask: Optional[torch.Tensor] = None, dtype=torch.float32) -> torch.Tensor:
    """Dense-row softmax over the layout (sparse_softmax.cu:113-155), blocks in, blocks out."""
    xs = x.detach().cpu().to(dtype)
    dense = to_dense(xs, pattern, block) * scale
    keep = _score_mask(pattern, block, causal, key_padding_mask, dense.shape[:-2])
    dense = dense.masked_fill(~keep, float("-inf"))
    mx = dense.amax(dim=-1, keepdim=True)
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)     # fully masked rows -> zeros
    e = torch.exp(dense - mx)
    s = e.sum(dim=-1, keepdim=True)
    y = torch.where(s > 0, e / s.clamp_min(torch.finfo(dtype).tiny), torch.zeros_like(e))
    return to_sparse(y, pattern, block).contiguous()


def softmax_backward(y: torch.Tensor, dy: torch.Tensor, pattern, block: int, scale: float = 1.0,
                     dtype=torch.float32) -> torch.Tensor:
    """dx = scale * y * (dy - sum_row(dy * y)) (sparse_softmax.cu:165-205 plus the fused scale)."""
    yd = to_dense(y.detach().cpu().to(dtype), pattern, block)
    dyd = to_dense(dy.detach().cpu().to(dtype), pattern, block)
    dot = (yd * dyd).sum(dim=-1, keepdim=True)
    dx = scale * yd * (dyd - dot)
    return to_sparse(dx, pattern, block).contiguous()


# --------------------------------------------------------------------------- literal replay of the reference softmax kernels
def _tree_sum_lane0(v: np.ndarray) -> np.ndarray:
    """Value lane 0 holds after ``for (offset = 16; offset > 0; offset /= 2) v += __shfl_down_sync(v, offset)``
    (sparse_softmax.cu:84-85, 98-99): fp32 additions in exactly that order.  ``v`` is [..., 32]."""
    v = v.astype(np.float32).copy()
    for offset in (16, 8, 4, 2, 1):
        shifted = v.copy()
        shifted[..., : 32 - offset] = v[..., offset:]       # lanes past the end read their own value
        v = (v + shifted).astype(np.float32)
    return v[..., 0]


def _row_blocks(row_blocks: np.ndarray, row_table: np.ndarray, block_row: int) -> np.ndarray:
    """Storage indices (the descriptors' first word) of the blocks of one block row, in layout order."""
    first, last = int(row_table[block_row]), int(row_table[block_row + 1])
    return np.asarray(row_blocks).reshape(-1, 2)[first:last, 0].astype(np.int64)


def _strided_partials(values: np.ndarray, reduce_max: bool) -> np.ndarray:
    """Per-thread partial results of the strided walk ``block_ptr = start + threadIdx.y; block_ptr += 32``
    (sparse_softmax.cu:26-33, 77-82).  ``values`` is [blocks, 32] (one dense row of every block of the row,
    index = threadIdx.x); returns [32 (threadIdx.y), 32 (threadIdx.x)] fp32."""
    out = np.full((32, 32), -1e5 if reduce_max else 0.0, dtype=np.float32)        # the seeds of :24 and :75
    for i in range(values.shape[0]):
        y = i % 32
        out[y] = np.maximum(out[y], values[i]) if reduce_max else (out[y] + values[i]).astype(np.float32)
    return out


def _block_reduce(values: np.ndarray, reduce_max: bool) -> np.float32:
    """reduce_sparse_matrix_32x32_row_max / _row_sum (sparse_softmax.cu:14-56, 63-105) for one dense row."""
    part = _strided_partials(values, reduce_max)
    if reduce_max:
        return np.float32(part.max())            # a maximum does not depend on the order of the tree
    per_warp = _tree_sum_lane0(part)             # [32]: shared[threadIdx.y]
    return np.float32(_tree_sum_lane0(per_warp[None, :])[0])


def reference_softmax_forward_emulated(x, row_blocks, row_table) -> np.ndarray:
    """sparse_softmax_32x32_forward_kernel (sparse_softmax.cu:113-155) replayed on the CPU in fp32.
    ``x`` is [batches, nnz, 32, 32]; the layout is the ROW layout in the int32 wire format."""
    x = np.asarray(x, dtype=np.float32)
    y = np.zeros_like(x)
    table = np.asarray(row_table)
    for z in range(x.shape[0]):
        for block_row in range(len(table) - 1):
            idx = _row_blocks(row_blocks, table, block_row)
            if len(idx) == 0:
                continue
            for offset_row in range(32):
                vals = x[z, idx, offset_row, :]                                  # [blocks, 32]
                mx = _block_reduce(vals, True)
                e = np.exp((vals - mx).astype(np.float32)).astype(np.float32)    # __expf(x - max), :139
                total = _block_reduce(e, False)
                with np.errstate(divide="ignore", invalid="ignore"):
                    y[z, idx, offset_row, :] = (e / total).astype(np.float32)    # :153
    return y


def reference_softmax_backward_emulated(y, dy, row_blocks, row_table) -> np.ndarray:
    """sparse_softmax_32x32_backward_kernel (sparse_softmax.cu:165-205) replayed on the CPU in fp32."""
    y = np.asarray(y, dtype=np.float32)
    dy = np.asarray(dy, dtype=np.float32)
    dx = np.zeros_like(y)
    table = np.asarray(row_table)
    for z in range(y.shape[0]):
        for block_row in range(len(table) - 1):
            idx = _row_blocks(row_blocks, table, block_row)
            if len(idx) == 0:
                continue
            for offset_row in range(32):
                yy, dd = y[z, idx, offset_row, :], dy[z, idx, offset_row, :]
                total = _block_reduce((dd * yy).astype(np.float32), False)       # :190, :193
                dx[z, idx, offset_row, :] = ((dd - total) * yy).astype(np.float32)   # :203
    return dx


# --------------------------------------------------------------------------- benchmark workload
def strided_local_pattern(size: int, stride: int = 8, window: int = 2) -> np.ndarray:
    """Block pattern of the benchmark workload: every ``stride``-th block diagonal plus a band of
    half-width ``window`` (non-causal), as an int64 0/1 array."""
    i = np.arange(size)[:, None]
    j = np.arange(size)[None, :]
    return ((((i - j) % stride) == 0) | (np.abs(i - j) <= window)).astype(np.int64)


# --------------------------------------------------------------------------- attention step
def attention_forward(q, k, v, pattern, block: int, scale: float, causal: bool = False, dtype=torch.float32):
    """SDD(Q K^T) -> softmax -> DSD(P V) for [..., seq, d] inputs; returns (out, probs_blocks)."""
    s = sparse_matmul(q, k, "sdd", pattern, block, False, True, dtype)
    p = softmax_forward(s, pattern, block, scale, causal, None, dtype)
    o = sparse_matmul(p, v, "dsd", pattern, block, False, False, dtype)
    return o, p


def attention_forward_dense(q, k, v, pattern, block: int, scale: float, causal: bool = False,
                            key_padding_mask: Optional[torch.Tensor] = None, dtype=torch.float32):
    """Masked dense attention forward: (out, lse) with lse = log sum exp of the scaled, masked scores
    per query row (-inf and a zero output row where every score is masked).  This is the composition
    sdd (sparse_smm_gpu.cu:22-99) -> softmax (sparse_softmax.cu:113-155) -> dsd (sparse_smm_gpu.cu:101-183)
    written densely."""
    q = q.detach().cpu().to(dtype)
    k = k.detach().cpu().to(dtype)
    v = v.detach().cpu().to(dtype)
    keep = _score_mask(pattern, block, causal, key_padding_mask, q.shape[:-2])
    scores = (q @ k.transpose(-1, -2)) * scale
    scores = scores.masked_fill(~keep, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    return probs @ v, lse


def attention_step_dense(q, k, v, do, pattern, block: int, scale: float, causal: bool = False,
                         dtype=torch.float32, key_padding_mask: Optional[torch.Tensor] = None):
    """Forward and backward of masked dense attention through torch autograd.

    Returns (out, dq, dk, dv); this is the CPU baseline computation: the same
    masked-dense work a user without block-sparse kernels would run.
    """
    q = q.detach().cpu().to(dtype).requires_grad_(True)
    k = k.detach().cpu().to(dtype).requires_grad_(True)
    v = v.detach().cpu().to(dtype).requires_grad_(True)
    keep = _score_mask(pattern, block, causal, key_padding_mask, q.shape[:-2])
    scores = (q @ k.transpose(-1, -2)) * scale
    # rows without any unmasked score: probabilities (and all their gradients) are zero
    dead = ~keep.any(dim=-1, keepdim=True)
    scores = scores.masked_fill(~keep & ~dead, float("-inf"))
    probs = torch.softmax(scores, dim=-1).masked_fill(dead, 0.0)
    out = probs @ v
    if do is None:
        return out.detach(), None, None, None
    out.backward(do.detach().cpu().to(dtype))
    return out.detach(), q.grad, k.grad, v.grad
