"""CPU tests: the oracle against the fixtures produced by executing the reference."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden_layout_names, load_golden_layout, seeded
from oracle import oracle


@pytest.mark.parametrize("name", golden_layout_names())
def test_layout_oracle_matches_reference_fixture(name):
    g = load_golden_layout(name)
    pattern = np.array(g["pattern"], dtype=np.int64)
    rb, rt = oracle.create_layout(pattern)
    cb, ct = oracle.create_layout(pattern, transpose=True)
    assert rb.dtype == np.int32 and rt.dtype == np.int32
    assert rb.tolist() == g["row_blocks"] and rt.tolist() == g["row_table"]
    assert cb.tolist() == g["col_blocks"] and ct.tolist() == g["col_table"]
    assert oracle.sparse_positions(pattern).tolist() == g["sparse_positions"]


def test_known_answer_from_reference_run():
    # 4x3 pattern executed through the reference's layout.py on CPU.
    g = load_golden_layout("kat_4x3")
    assert g["row_blocks"] == [0, 0, 1, 2, 2, 65537, 3, 131072, 4, 131073, 5, 196610]
    assert g["row_table"] == [0, 2, 3, 5, 6]
    assert g["col_blocks"] == [0, 0, 3, 131072, 2, 65537, 4, 131073, 1, 2, 5, 196610]
    assert g["col_table"] == [0, 2, 4, 6]


@pytest.mark.parametrize("dtype", [np.uint8, np.int32, np.float32, np.bool_])
def test_layout_oracle_pattern_dtypes(dtype):
    g = load_golden_layout("empty_row_col_5x4")
    pattern = np.array(g["pattern"]).astype(dtype)
    rb, rt = oracle.create_layout(pattern)
    assert rb.tolist() == g["row_blocks"] and rt.tolist() == g["row_table"]


def _dense_reference(a, b, mode, pattern, block, ta, tb):
    """Independent dense autograd model: plain matmul with a hard mask."""
    mask = oracle.element_mask(pattern, block).double()
    ad = oracle.to_dense(a, pattern, block) if mode[1] == "s" else a
    bd = oracle.to_dense(b, pattern, block) if mode[2] == "s" else b
    c = (ad.transpose(-1, -2) if ta else ad) @ (bd.transpose(-1, -2) if tb else bd)
    return c * mask if mode[0] == "s" else c


def _operands(mode, ta, tb, pattern, block, inner, seed):
    rows, cols = pattern.shape[0] * block, pattern.shape[1] * block
    nnz = int((pattern != 0).sum())
    if mode == "sdd":
        m, n, k = rows, cols, inner
    elif mode == "dsd":
        m, k, n = (cols, rows, inner) if ta else (rows, cols, inner)
    else:
        k, n, m = (cols, rows, inner) if tb else (rows, cols, inner)
    a_shape = (2, nnz, block, block) if mode[1] == "s" else ((2, k, m) if ta else (2, m, k))
    b_shape = (2, nnz, block, block) if mode[2] == "s" else ((2, n, k) if tb else (2, k, n))
    return seeded(a_shape, seed).double(), seeded(b_shape, seed + 1).double()


@pytest.mark.parametrize("mode", ["sdd", "dsd", "dds"])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_matmul_oracle_equals_dense_and_reference_backward_table(mode, ta, tb):
    """The oracle run through the call sequence the REFERENCE's backward issues
    (fixture autograd_table.json) gives the gradients of dense autograd."""
    pattern = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 0], [0, 0, 1]])
    block = 4  # the oracle is block-size agnostic; small keeps this fast
    a, b = _operands(mode, ta, tb, pattern, block, 8, 7)
    a.requires_grad_(True)
    b.requires_grad_(True)
    ref = _dense_reference(a, b, mode, pattern, block, ta, tb)
    got = oracle.sparse_matmul(a, b, mode, pattern, block, ta, tb, dtype=torch.float64)
    got_dense = oracle.to_dense(got, pattern, block) if mode[0] == "s" else got
    assert torch.allclose(got_dense, ref.detach(), atol=1e-12)

    dc = seeded(tuple(got.shape), 11).double()
    dc_dense = oracle.to_dense(dc, pattern, block) if mode[0] == "s" else dc
    ref.backward(dc_dense)
    with open(os.path.join(GOLDEN, "autograd_table.json")) as f:
        table = json.load(f)["table"]
    row = next(r for r in table if r["forward"] == {"mode": mode, "trans_a": ta, "trans_b": tb})
    tensors = {"a": a.detach(), "b": b.detach(), "dc": dc}
    for name, grad in (("da", a.grad), ("db", b.grad)):
        call = row[name]
        out = oracle.sparse_matmul(tensors[call["a"]], tensors[call["b"]], call["mode"], pattern, block,
                                   call["trans_a"], call["trans_b"], dtype=torch.float64)
        if call["mode"][0] == "s":
            # gradients of a sparse operand only exist inside the layout
            grad = oracle.to_sparse(oracle.to_dense(grad, pattern, block), pattern, block) \
                if grad.dim() == 4 else oracle.to_sparse(grad, pattern, block)
        assert torch.allclose(out, grad, atol=1e-10), name


def test_softmax_oracle_properties():
    pattern = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 0]])
    block = 4
    nnz = int(pattern.sum())
    x = seeded((2, nnz, block, block), 3).double().requires_grad_(True)
    dense = oracle.to_dense(x, pattern, block) * 0.5
    keep = oracle.element_mask(pattern, block)
    y_ref = torch.softmax(dense.masked_fill(~keep, float("-inf")), dim=-1)
    y = oracle.softmax_forward(x, pattern, block, scale=0.5, dtype=torch.float64)
    assert torch.allclose(oracle.to_dense(y, pattern, block), y_ref.detach(), atol=1e-12)
    assert torch.allclose(oracle.to_dense(y, pattern, block).sum(-1), torch.ones(2, 12, dtype=torch.float64))
    dy = seeded(tuple(y.shape), 5).double()
    y_ref.backward(oracle.to_dense(dy, pattern, block))
    dx = oracle.softmax_backward(y, dy, pattern, block, scale=0.5, dtype=torch.float64)
    assert torch.allclose(dx, x.grad, atol=1e-12)


def test_softmax_oracle_masks():
    pattern = np.array([[1, 1], [1, 1]])
    block = 4
    x = seeded((2, 4, block, block), 9).double()
    y = oracle.to_dense(oracle.softmax_forward(x, pattern, block, causal=True, dtype=torch.float64), pattern, block)
    assert torch.all(torch.triu(y, diagonal=1) == 0)
    assert torch.allclose(y.sum(-1), torch.ones(2, 8, dtype=torch.float64))
    kpm = torch.zeros(2, 8, dtype=torch.bool)
    kpm[0, 3:] = True
    kpm[1, :] = True        # a fully padded batch entry gives all-zero rows
    y = oracle.to_dense(oracle.softmax_forward(x, pattern, block, key_padding_mask=kpm, dtype=torch.float64),
                        pattern, block)
    assert torch.all(y[0, :, 3:] == 0) and torch.allclose(y[0].sum(-1), torch.ones(8, dtype=torch.float64))
    assert torch.all(y[1] == 0)


# ---- the softmax definition against a literal replay of the reference kernels' arithmetic
# (sparse_softmax.cu:14-56, 63-105, 113-155, 165-205): scale 1, no masks, block 32, fp32
@pytest.mark.parametrize("name", ["kat_4x3", "empty_row_col_5x4"])
def test_softmax_definition_equals_reference_kernel_replay(name):
    g = load_golden_layout(name)
    pattern = np.array(g["pattern"], dtype=np.int64)
    nnz = int(pattern.sum())
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(2, nnz, 32, 32, generator=gen) * 3.0
    dy = torch.randn(2, nnz, 32, 32, generator=gen)
    y_def = oracle.softmax_forward(x, pattern, 32)
    y_ref = oracle.reference_softmax_forward_emulated(x.numpy(), g["row_blocks"], g["row_table"])
    assert np.abs(y_def.numpy() - y_ref).max() <= 1e-6
    # every dense row that has blocks sums to 1 in the replay too
    dense = oracle.to_dense(torch.from_numpy(y_ref), pattern, 32)
    has_blocks = torch.as_tensor(pattern.sum(axis=1) > 0).repeat_interleave(32)
    assert torch.allclose(dense.sum(-1)[:, has_blocks], torch.ones(2, int(has_blocks.sum())), atol=1e-5)
    dx_def = oracle.softmax_backward(y_def, dy, pattern, 32)
    dx_ref = oracle.reference_softmax_backward_emulated(y_ref, dy.numpy(), g["row_blocks"], g["row_table"])
    assert np.abs(dx_def.numpy() - dx_ref).max() <= 1e-6


def test_softmax_definition_and_reference_part_ways_below_the_seed():
    """The reference seeds its row maximum with -1e5 (sparse_softmax.cu:24).  A row whose every score lies
    below that keeps the seed as its maximum, all exponentials underflow and the row becomes 0 / 0; the
    masked dense definition (and the kernels of this library) subtract the true maximum and return the
    proper probabilities.  Rows above the seed agree."""
    g = load_golden_layout("kat_4x3")
    pattern = np.array(g["pattern"], dtype=np.int64)
    nnz = int(pattern.sum())
    x = torch.randn(1, nnz, 32, 32, generator=torch.Generator().manual_seed(3))
    rows_blocks = np.asarray(g["row_blocks"]).reshape(-1, 2)
    first_row_blocks = rows_blocks[g["row_table"][0]:g["row_table"][1], 0]
    x[0, first_row_blocks, 5, :] -= 2.0e5                     # dense row 5 of block row 0: everything below -1e5
    y_def = oracle.softmax_forward(x, pattern, 32).numpy()
    y_ref = oracle.reference_softmax_forward_emulated(x.numpy(), g["row_blocks"], g["row_table"])
    low = y_ref[0, first_row_blocks, 5, :]
    assert not np.isfinite(low).all() or np.abs(low).max() == 0.0          # 0 / 0 in the reference's arithmetic
    assert abs(y_def[0, first_row_blocks, 5, :].sum() - 1.0) <= 1e-5       # a probability row in the definition
    keep = np.ones_like(y_ref, dtype=bool)
    keep[0, first_row_blocks, 5, :] = False
    assert np.abs(y_def[keep] - y_ref[keep]).max() <= 1e-6
