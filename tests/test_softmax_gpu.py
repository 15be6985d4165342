"""GPU parity of the block-sparse softmax (forward, backward, masks) against the CPU oracle.
Tolerance: max |got - ref| / max |ref| <= 1e-4 (fp32), 1e-2 (fp16), 3e-2 (bf16)."""
import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden_layout, seeded
from oracle import oracle

pytestmark = pytest.mark.gpu


def _layout(pattern, block):
    from sparse import SparseLayout
    return SparseLayout(torch.as_tensor(np.asarray(pattern)), block=block)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block", [16, 32, 64, 128])
@pytest.mark.parametrize("name", ["kat_4x3", "empty_row_col_5x4", "one_by_one"])
def test_forward_backward_matches_oracle(dtype, block, name):
    from sparse import softmax
    pattern = np.array(load_golden_layout(name)["pattern"])
    layout = _layout(pattern, block)
    nnz = int(pattern.sum())
    x = seeded((2, 3, nnz, block, block), 31, dtype)
    xg = x.cuda().requires_grad_(True)
    y = softmax(xg, layout, scale=0.7)
    ref = oracle.softmax_forward(x, pattern, block, scale=0.7)
    assert y.dtype == dtype
    assert_close(y, ref, dtype, "softmax forward")
    dy = seeded(tuple(y.shape), 33, dtype)
    y.backward(dy.cuda())
    dref = oracle.softmax_backward(y.detach().cpu(), dy, pattern, block, scale=0.7)
    assert_close(xg.grad, dref, dtype, "softmax backward")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("block", [16, 32, 64])
def test_causal_and_key_padding_masks(dtype, block):
    from sparse import softmax
    from sparse.patterns import local_global_causal
    pattern = local_global_causal(6, 3, 1).numpy()
    layout = _layout(pattern, block)
    nnz = int(pattern.sum())
    x = seeded((2, 2, nnz, block, block), 41, dtype)
    y = softmax(x.cuda(), layout, scale=0.125, causal=True)
    assert_close(y, oracle.softmax_forward(x, pattern, block, 0.125, True), dtype, "causal")
    dense = layout.to_dense(y).float().cpu()
    assert torch.all(torch.triu(dense, diagonal=1) == 0)
    assert torch.allclose(dense.sum(-1), torch.ones_like(dense.sum(-1)), atol=2e-2 if dtype != torch.float32 else 1e-5)

    kpm = torch.zeros(2, 6 * block, dtype=torch.bool)
    kpm[0, 5 * block + 3:] = True
    kpm[1, : 2 * block + 1] = True      # rows that only see the first blocks become fully masked
    y = softmax(x.cuda(), layout, scale=0.125, causal=True, key_padding_mask=kpm.cuda())
    ref = oracle.softmax_forward(x, pattern, block, 0.125, True, kpm)
    assert_close(y, ref, dtype, "causal + key padding")
    assert torch.isfinite(y).all()


def test_fully_masked_rows_give_zero():
    from sparse import softmax
    pattern = np.ones((2, 2), dtype=np.int64)
    layout = _layout(pattern, 32)
    x = seeded((1, 4, 32, 32), 43)
    kpm = torch.ones(1, 64, dtype=torch.bool)
    y = softmax(x.cuda(), layout, key_padding_mask=kpm.cuda())
    assert torch.all(y == 0)


@pytest.mark.parametrize("dtype,block,cols", [(torch.float16, 32, 80), (torch.float32, 32, 70),
                                               (torch.float16, 64, 300), (torch.float32, 64, 140)])
def test_long_rows_take_wide_teams_and_streaming_path(dtype, block, cols):
    """Rows spanning many blocks: teams wider than a warp, and (last two cases) rows longer than the
    register-resident limit of 2048 16-byte chunks."""
    from sparse import softmax
    pattern = np.zeros((2, cols), dtype=np.int64)
    pattern[0, :] = 1
    pattern[1, ::3] = 1
    layout = _layout(pattern, block)
    nnz = int(pattern.sum())
    x = seeded((1, nnz, block, block), 47, dtype)
    xg = x.cuda().requires_grad_(True)
    y = softmax(xg, layout, scale=1.3)
    assert_close(y, oracle.softmax_forward(x, pattern, block, 1.3), dtype, "long rows forward")
    dy = seeded(tuple(y.shape), 49, dtype)
    y.backward(dy.cuda())
    assert_close(xg.grad, oracle.softmax_backward(y.detach().cpu(), dy, pattern, block, 1.3), dtype,
                 "long rows backward")


def test_large_logits_are_stable():
    from sparse import softmax
    pattern = np.array([[1, 1, 0], [0, 1, 1]])
    layout = _layout(pattern, 32)
    x = seeded((1, 4, 32, 32), 51) * 200.0
    y = softmax(x.cuda(), layout)
    assert torch.isfinite(y).all()
    assert_close(y, oracle.softmax_forward(x, pattern, 32, dtype=torch.float64), torch.float32, "large logits")
