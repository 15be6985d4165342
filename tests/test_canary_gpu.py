"""Out-of-bounds write check without a sanitizer: every output buffer of the C-ABI entry points sits
between two guard regions filled with a sentinel; after the call the guards must be untouched and
the output must equal the one computed into a plain buffer.  Covers the three matmul engines (tcgen05
block 64 and block 32, CUDA cores), every mode, the softmax forward / backward and the fused
attention forward and backward, on a layout with an empty block row and an empty block column."""
import ctypes
import os

import pytest
import torch

from conftest import PKG, load_golden_layout

pytestmark = pytest.mark.gpu

GUARD = 4096          # elements on either side
MATMUL_ARGS = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 6 + \
    [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]


def _library():
    lib = ctypes.CDLL(os.path.join(PKG, "libbsa_b200.so"))
    lib.bsa_matmul.argtypes = MATMUL_ARGS
    lib.bsa_softmax_forward.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    lib.bsa_softmax_backward.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_int64, ctypes.c_void_p]
    lib.bsa_attention_forward.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_int64] * 5 + \
        [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.bsa_attention_backward.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 13 + [ctypes.c_int64] * 5 + \
        [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.bsa_workspace_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib


class Guarded:
    """An output tensor of `shape` inside a larger allocation whose margins hold a sentinel."""

    def __init__(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        self.sentinel = 123.0 if dtype != torch.float32 else 12345.0
        self.raw = torch.full((n + 2 * GUARD,), self.sentinel, device="cuda", dtype=dtype)
        self.view = self.raw[GUARD:GUARD + n].view(shape)
        self.view.fill_(float("nan"))

    def check(self, what):
        torch.cuda.synchronize()
        assert bool((self.raw[:GUARD] == self.sentinel).all()), "%s wrote below its output" % what
        assert bool((self.raw[-GUARD:] == self.sentinel).all()), "%s wrote above its output" % what
        assert not bool(torch.isnan(self.view.float()).any()), "%s left part of its output unwritten" % what


@pytest.mark.parametrize("block,dtype,engine", [(64, torch.float16, 2), (32, torch.float32, 2), (32, torch.float16, 2),
                                                (64, torch.float32, 1), (128, torch.float16, 1)])
@pytest.mark.parametrize("mode", ["sdd", "dsd", "dds"])
def test_matmul_writes_only_its_output(block, dtype, engine, mode):
    from sparse import SparseLayout
    lib = _library()
    pattern = torch.tensor(load_golden_layout("empty_row_col_5x4")["pattern"])
    layout = SparseLayout(pattern, block=block)
    rows, cols = pattern.shape[0] * block, pattern.shape[1] * block
    nnz, z, d = layout.num_blocks, 3, 64
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    gen = torch.Generator(device="cuda").manual_seed(3)
    rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=gen).to(dtype)
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    if mode == "sdd":       # blocks = A[rows, d] . B[cols, d]^T
        a, b, out_shape = rnd(z, rows, d), rnd(z, cols, d), (z, nnz, block, block)
        m, n, k, flags, (blk, tab) = rows, cols, d, (0, 0, 1), layout.row_layout
    elif mode == "dsd":     # C[rows, d] = blocks . B[cols, d]
        a, b, out_shape = rnd(z, nnz, block, block), rnd(z, cols, d), (z, rows, d)
        m, n, k, flags, (blk, tab) = rows, d, cols, (1, 0, 0), layout.row_layout
    else:                   # C[d, cols] = A[rows, d]^T . blocks
        a, b, out_shape = rnd(z, rows, d), rnd(z, nnz, block, block), (z, d, cols)
        m, n, k, flags, (blk, tab) = d, cols, rows, (2, 1, 0), layout.col_layout
    out = Guarded(out_shape, dtype)
    st = lib.bsa_matmul(flags[0], code, flags[1], flags[2], a.data_ptr(), b.data_ptr(), out.view.data_ptr(),
                        blk.data_ptr(), tab.data_ptr(), nnz, tab.numel() - 1, z, m, n, k, block,
                        ws.data_ptr(), 256, engine, stream)
    assert st == 0, st
    out.check("%s block %d %s engine %d" % (mode, block, dtype, engine))
    assert lib.bsa_workspace_status(ws.data_ptr(), stream) == 0
    from sparse.kernel import sparse_ops
    names = {1: "simt", 2: "tcgen05"}
    ref = sparse_ops.sparse_matmul(a, b, mode, layout.row_layout, layout.col_layout, bool(flags[1]), bool(flags[2]),
                                   block, names[engine])
    assert torch.equal(out.view, ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_softmax_and_attention_write_only_their_outputs(dtype):
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    lib = _library()
    pattern = torch.tensor(load_golden_layout("empty_row_col_5x4")["pattern"])
    block = 64
    layout = SparseLayout(pattern, block=block)
    nnz, z = layout.num_blocks, 4
    code = {torch.float32: 0, torch.float16: 1}[dtype]
    blk, tab = layout.row_layout
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(z, nnz, block, block, device="cuda", generator=gen).to(dtype)
    dy = torch.randn(z, nnz, block, block, device="cuda", generator=gen).to(dtype)
    y = Guarded((z, nnz, block, block), dtype)
    st = lib.bsa_softmax_forward(code, x.data_ptr(), y.view.data_ptr(), blk.data_ptr(), tab.data_ptr(), nnz,
                                 pattern.shape[0], z, block, 0.5, 0, None, 0, 0, layout.max_row_blocks, stream)
    assert st == 0, st
    y.check("softmax forward")
    assert torch.equal(y.view, sparse_ops.sparse_softmax_forward(x, blk, tab, 0.5, False, None, layout.max_row_blocks))
    dx = Guarded((z, nnz, block, block), dtype)
    st = lib.bsa_softmax_backward(code, y.view.data_ptr(), dy.data_ptr(), dx.view.data_ptr(), blk.data_ptr(),
                                  tab.data_ptr(), nnz, pattern.shape[0], z, block, 0.5, layout.max_row_blocks, stream)
    assert st == 0, st
    dx.check("softmax backward")
    if dtype != torch.float16:
        return
    d = 128
    q = torch.randn(z, pattern.shape[0] * block, d, device="cuda", generator=gen).half()
    k = torch.randn(z, pattern.shape[1] * block, d, device="cuda", generator=gen).half()
    v = torch.randn(z, pattern.shape[1] * block, d, device="cuda", generator=gen).half()
    o = Guarded((z, pattern.shape[0] * block, d), torch.float16)
    lse = Guarded((z, pattern.shape[0] * block), torch.float32)
    lse.view.fill_(0.0)            # (-inf is a legal value of this output)
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    st = lib.bsa_attention_forward(1, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.view.data_ptr(), lse.view.data_ptr(),
                                   blk.data_ptr(), tab.data_ptr(), nnz, pattern.shape[0], pattern.shape[1], z, d, block,
                                   0.1, 0, None, 0, 0, 0, ws.data_ptr(), 256, stream)
    assert st == 0, st
    o.check("attention forward output")
    torch.cuda.synchronize()
    assert bool((lse.raw[:GUARD] == lse.sentinel).all()) and bool((lse.raw[-GUARD:] == lse.sentinel).all())
    assert lib.bsa_workspace_status(ws.data_ptr(), stream) == 0
    # fused backward: three gradient outputs and the statistics scratch
    do = torch.randn(z, pattern.shape[0] * block, d, device="cuda", generator=gen).half()
    cblk, ctab = layout.col_layout
    dq = Guarded((z, pattern.shape[0] * block, d), torch.float16)
    dk = Guarded((z, pattern.shape[1] * block, d), torch.float16)
    dv = Guarded((z, pattern.shape[1] * block, d), torch.float16)
    stats = Guarded((z, pattern.shape[0] * block, 2), torch.float32)
    st = lib.bsa_attention_backward(1, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.view.data_ptr(), do.data_ptr(),
                                    lse.view.data_ptr(), dq.view.data_ptr(), dk.view.data_ptr(), dv.view.data_ptr(),
                                    blk.data_ptr(), tab.data_ptr(), cblk.data_ptr(), ctab.data_ptr(),
                                    nnz, pattern.shape[0], pattern.shape[1], z, d, block, 0.1, 0, None, 0, 0, 0,
                                    stats.view.data_ptr(), stats.view.numel() * 4, ws.data_ptr(), 256, stream)
    assert st == 0, st
    dq.check("attention backward dQ")
    dk.check("attention backward dK")
    dv.check("attention backward dV")
    torch.cuda.synchronize()
    assert bool((stats.raw[:GUARD] == stats.sentinel).all()) and bool((stats.raw[-GUARD:] == stats.sentinel).all())
    assert lib.bsa_workspace_status(ws.data_ptr(), stream) == 0
    got = sparse_ops.sparse_attention_backward(q, k, v, o.view, do, lse.view, blk, tab, cblk, ctab, block, 0.1, False, None)
    assert torch.equal(dq.view, got[0]) and torch.equal(dk.view, got[1]) and torch.equal(dv.view, got[2])
