"""GPU parity: layout metadata built on the device is bit-exact against the
fixtures produced by the reference's own layout.py and against the oracle."""
import numpy as np
import pytest
import torch

from conftest import golden_layout_names, load_golden_layout
from oracle import oracle

pytestmark = pytest.mark.gpu


def _check(layout, row_blocks, row_table, col_blocks, col_table):
    for t in layout.row_layout + layout.col_layout:
        assert t.dtype == torch.int32 and t.is_cuda and t.is_contiguous()
    assert layout.row_layout[0].cpu().tolist() == list(row_blocks)
    assert layout.row_layout[1].cpu().tolist() == list(row_table)
    assert layout.col_layout[0].cpu().tolist() == list(col_blocks)
    assert layout.col_layout[1].cpu().tolist() == list(col_table)


@pytest.mark.parametrize("name", golden_layout_names())
def test_device_layout_matches_reference_fixture(name):
    from sparse import SparseLayout
    g = load_golden_layout(name)
    layout = SparseLayout(torch.tensor(g["pattern"]))
    _check(layout, g["row_blocks"], g["row_table"], g["col_blocks"], g["col_table"])
    assert layout.sparse_positions.tolist() == g["sparse_positions"]
    assert layout.block == 32


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.uint8, torch.float32, torch.bool, torch.float16])
def test_device_layout_pattern_dtypes(dtype):
    from sparse import SparseLayout
    g = load_golden_layout("empty_row_col_5x4")
    for device in ("cpu", "cuda"):
        layout = SparseLayout(torch.tensor(g["pattern"]).to(dtype).to(device), block=64)
        _check(layout, g["row_blocks"], g["row_table"], g["col_blocks"], g["col_table"])


@pytest.mark.parametrize("rows,cols,density,seed", [(1, 1, 1.0, 0), (7, 300, 0.3, 1), (300, 7, 0.3, 2),
                                                    (257, 1100, 0.05, 3), (1100, 1030, 0.5, 4), (64, 64, 0.0, 5)])
def test_device_layout_random_patterns_match_oracle(rows, cols, density, seed):
    from sparse import SparseLayout
    gen = torch.Generator().manual_seed(seed)
    pattern = (torch.rand(rows, cols, generator=gen) < density).long()
    layout = SparseLayout(pattern)
    rb, rt = oracle.create_layout(pattern.numpy())
    cb, ct = oracle.create_layout(pattern.numpy(), transpose=True)
    _check(layout, rb.tolist(), rt.tolist(), cb.tolist(), ct.tolist())
    assert layout.num_blocks == int(pattern.sum())


def test_converters_roundtrip():
    from sparse import SparseLayout
    g = load_golden_layout("kat_4x3")
    pattern = torch.tensor(g["pattern"])
    for block in (16, 32, 64):
        layout = SparseLayout(pattern, block=block)
        x = torch.randn(2, 3, 4 * block, 3 * block, device="cuda", dtype=torch.float16)
        s = layout.to_sparse(x)
        assert s.shape == (2, 3, 6, block, block)
        assert torch.equal(s.cpu(), oracle.to_sparse(x.cpu(), pattern.numpy(), block))
        d = layout.to_dense(s)
        mask = oracle.element_mask(pattern.numpy(), block)
        assert torch.equal(d.cpu(), x.cpu() * mask)
        # CPU tensors take the pure torch path with the same result
        assert torch.equal(layout.to_sparse(x.cpu()), s.cpu())
        assert torch.equal(layout.to_dense(s.cpu()), d.cpu())
