"""GPU test of bsa_matmul_noalloc, the entry point for callers that cannot allocate device
memory (a plugin living inside another framework's pool, a loop that must never hit cudaMalloc).
It keeps the kernels' scratch words in a static device array instead of taking a workspace.

The test drives both entry points through the C ABI with ctypes: the product computed through
bsa_matmul_noalloc must equal the one computed through bsa_matmul (caller-provided workspace)
within the tolerance the matmul tests use, on two calls in a row -- the second call sees the
static array as the first one left it.  One product is also compared with the CPU oracle, so the
file stands on its own; the asynchronous mode (wait_and_check = 0) is followed by the status
accessor; and the free device memory reported by the driver must not shrink across the calls.
This file sorts last so a run that stops at the first failure has already executed every other test.
"""
import ctypes
import os

import pytest
import torch

from conftest import PKG, TOL, rel_err

pytestmark = pytest.mark.gpu

MATMUL_ARGS = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 6 + [ctypes.c_int]


def _library():
    lib = ctypes.CDLL(os.path.join(PKG, "libbsa_b200.so"))
    lib.bsa_matmul.argtypes = MATMUL_ARGS + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    lib.bsa_matmul_noalloc.argtypes = MATMUL_ARGS + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.bsa_workspace_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.bsa_matmul_noalloc_status.argtypes = [ctypes.c_void_p]
    return lib


@pytest.mark.parametrize("mode,engine", [("sdd", 2), ("dsd", 2), ("sdd", 1)])
def test_noalloc_entry_matches_workspace_entry_twice(mode, engine):
    from sparse import SparseLayout
    from sparse.patterns import strided_local
    lib = _library()
    torch.cuda.set_device(0)
    block, rows, dim, z = 64, 16, 64, 20
    layout = SparseLayout(strided_local(rows, 4, 1), block=block)
    nnz = layout.num_blocks
    blocks, table = layout.row_layout
    stream = torch.cuda.current_stream().cuda_stream
    workspace = torch.zeros(256, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(5)
    for call in range(2):
        if mode == "sdd":      # C_blocks = Q . K^T
            a = torch.randn(z, rows * block, dim, device="cuda", generator=gen).half()
            b = torch.randn(z, rows * block, dim, device="cuda", generator=gen).half()
            out_shape, sizes, flags = (z, nnz, block, block), (rows * block, rows * block, dim), (0, 0, 1)
        else:                  # C = P_blocks . V
            a = torch.rand(z, nnz, block, block, device="cuda", generator=gen).half()
            b = torch.randn(z, rows * block, dim, device="cuda", generator=gen).half()
            out_shape, sizes, flags = (z, rows * block, dim), (rows * block, dim, rows * block), (1, 0, 0)
        want = torch.empty(out_shape, device="cuda", dtype=torch.float16)
        got = torch.full(out_shape, float("nan"), device="cuda", dtype=torch.float16)
        common = (flags[0], 1, flags[1], flags[2], a.data_ptr(), b.data_ptr())
        tail = (blocks.data_ptr(), table.data_ptr(), nnz, table.numel() - 1, z, *sizes, block)
        st = lib.bsa_matmul(*common, want.data_ptr(), *tail, workspace.data_ptr(), 256, engine, stream)
        assert st == 0, st
        assert lib.bsa_workspace_status(workspace.data_ptr(), stream) == 0
        st = lib.bsa_matmul_noalloc(*common, got.data_ptr(), *tail, engine, 1, stream)
        assert st == 0, "bsa_matmul_noalloc returned %d on call %d" % (st, call)
        torch.cuda.synchronize()
        assert rel_err(got, want) <= TOL[torch.float16], "call %d differs" % call
        if call == 1 and mode == "sdd":
            # against the CPU oracle as well (first two batch entries)
            from oracle import oracle
            ref = oracle.sparse_matmul(a[:2].cpu(), b[:2].cpu(), "sdd", layout.pattern.numpy(), block, False, True)
            assert rel_err(got[:2], ref) <= TOL[torch.float16]


def test_noalloc_entry_async_mode_and_no_allocation():
    """wait_and_check = 0 returns right after the launch; the status accessor then synchronises and reports.
    The driver's free-memory figure is the same before and after the calls (nothing was allocated)."""
    from sparse import SparseLayout
    from sparse.patterns import strided_local
    lib = _library()
    torch.cuda.set_device(0)
    block, rows, dim, z = 64, 8, 64, 4
    layout = SparseLayout(strided_local(rows, 4, 1), block=block)
    nnz = layout.num_blocks
    blocks, table = layout.row_layout
    stream = torch.cuda.current_stream().cuda_stream
    a = torch.randn(z, rows * block, dim, device="cuda").half()
    b = torch.randn(z, rows * block, dim, device="cuda").half()
    got = torch.empty(z, nnz, block, block, device="cuda", dtype=torch.float16)
    args = (0, 1, 0, 1, a.data_ptr(), b.data_ptr(), got.data_ptr(), blocks.data_ptr(), table.data_ptr(), nnz,
            table.numel() - 1, z, rows * block, rows * block, dim, block, 0)
    assert lib.bsa_matmul_noalloc(*args, 1, stream) == 0          # first call on the device: address look-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert lib.bsa_matmul_noalloc(*args, 0, stream) == 0
        assert lib.bsa_matmul_noalloc_status(stream) == 0
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before
    from oracle import oracle
    ref = oracle.sparse_matmul(a[:1].cpu(), b[:1].cpu(), "sdd", layout.pattern.numpy(), block, False, True)
    assert rel_err(got[:1], ref) <= TOL[torch.float16]


def test_noalloc_entry_validates_like_the_workspace_entry():
    lib = _library()
    # rejected on the host before anything is launched (fake pointers are never dereferenced)
    assert lib.bsa_matmul_noalloc(3, 1, 0, 0, 16, 16, 16, 16, 16, 1, 1, 1, 64, 64, 64, 64, 0, 0, None) == 2
    assert lib.bsa_matmul_noalloc(0, 1, 0, 0, None, 16, 16, 16, 16, 1, 1, 1, 64, 64, 64, 64, 0, 0, None) == 1
