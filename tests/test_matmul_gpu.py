"""GPU parity of the block-sparse matmul against the masked dense CPU oracle.

Tolerance (stated by the parity contract): max |got - ref| / max |ref| <= 1e-4
for fp32 and <= 1e-2 for fp16 (bf16: 3e-2), ref = dense CPU torch computation
masked by the same layout on the same seeded inputs.
"""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden_layout, seeded
from oracle import oracle

pytestmark = pytest.mark.gpu

VARIANTS = [(m, ta, tb) for m in ("sdd", "dsd", "dds") for ta in (False, True) for tb in (False, True)]


def operands(mode, ta, tb, pattern, block, inner, batch, seed, dtype, dist="normal"):
    """Seeded CPU operands for op(A)[m,k] @ op(B)[k,n]; `inner` is the free dense size."""
    rows, cols = pattern.shape[0] * block, pattern.shape[1] * block
    nnz = int((np.asarray(pattern) != 0).sum())
    if mode == "sdd":
        m, n, k = rows, cols, inner
    elif mode == "dsd":
        m, k, n = (cols, rows, inner) if ta else (rows, cols, inner)
    else:
        k, n, m = (cols, rows, inner) if tb else (rows, cols, inner)
    a_shape = batch + ((nnz, block, block) if mode[1] == "s" else ((k, m) if ta else (m, k)))
    b_shape = batch + ((nnz, block, block) if mode[2] == "s" else ((n, k) if tb else (k, n)))
    return seeded(a_shape, seed, dtype, dist), seeded(b_shape, seed + 1, dtype, dist)


def run_case(mode, ta, tb, pattern, block, inner, dtype, engine, batch=(2,), seed=0, dist="normal"):
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    pattern = np.asarray(pattern)
    layout = SparseLayout(torch.as_tensor(pattern), block=block)
    a, b = operands(mode, ta, tb, pattern, block, inner, batch, seed, dtype, dist)
    got = sparse_ops.sparse_matmul(a.cuda(), b.cuda(), mode, layout.row_layout, layout.col_layout, ta, tb,
                                   block, engine)
    torch.cuda.synchronize()
    sparse_ops.check_device_status(0)
    ref = oracle.sparse_matmul(a, b, mode, pattern, block, ta, tb,
                               dtype=torch.float64 if dtype == torch.float32 else torch.float32)
    assert got.dtype == dtype and tuple(got.shape) == tuple(ref.shape)
    assert_close(got, ref, dtype, "%s ta=%s tb=%s block=%d %s %s" % (mode, ta, tb, block, dtype, engine))
    return got


def engines_for(dtype, block, inner):
    """Every case runs on the CUDA-core engine and on whatever `auto` selects (tcgen05 where it applies)."""
    return ["simt", "auto"]


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_all_variants_nonsquare_block32(mode, ta, tb, dtype):
    g = load_golden_layout("kat_4x3")
    for engine in engines_for(dtype, 32, 64):
        run_case(mode, ta, tb, g["pattern"], 32, 64, dtype, engine, seed=3)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_all_variants_nonsquare_block64(mode, ta, tb, dtype):
    g = load_golden_layout("empty_row_col_5x4")   # has an empty block row and an empty block column
    for inner in (64, 128):
        for engine in engines_for(dtype, 64, inner):
            run_case(mode, ta, tb, g["pattern"], 64, inner, dtype, engine, seed=5)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
def test_all_variants_block128_and_odd_inner(mode, ta, tb):
    run_case(mode, ta, tb, [[1, 0], [1, 1]], 128, 64, torch.float16, "auto", batch=(1,), seed=7)
    run_case(mode, ta, tb, [[1, 0, 1], [0, 1, 1]], 32, 40, torch.float32, "auto", batch=(1, 2), seed=9)


@pytest.mark.parametrize("name", ["single_block_3x3", "full_3x5", "one_by_one"])
@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
def test_edge_layouts(name, mode, ta, tb):
    g = load_golden_layout(name)
    for dtype, block in ((torch.float32, 32), (torch.float16, 64)):
        for engine in engines_for(dtype, block, 64):
            run_case(mode, ta, tb, g["pattern"], block, 64, dtype, engine, batch=(3,), seed=11)


def _wide_pattern():
    """40 x 48 blocks, about 30 % full, with a full row (48 blocks: several accumulations and more than
    one 32-descriptor window), a full column and an empty row."""
    rng = np.random.default_rng(0)
    pattern = (rng.random((40, 48)) < 0.3).astype(np.int64)
    pattern[3, :] = 1
    pattern[:, 5] = 1
    pattern[7, :] = 0
    return pattern


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_block32_on_tensor_cores(mode, ta, tb, dtype):
    """Block 32 on the tcgen05 engine, requested explicitly (it must not fall back): 16-bit types and
    fp32 as a 3xTF32 split, dense sizes that leave partial slices (96, 160) and the minimum (32)."""
    pattern = _wide_pattern()
    for inner in (32, 96, 160):
        run_case(mode, ta, tb, pattern, 32, inner, dtype, "tcgen05", batch=(2,), seed=31 + inner)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_block16_and_block128(mode, ta, tb, dtype):
    """The smallest and the largest block size: 16 (two blocks per 32-wide tile of the CUDA-core engine)
    and 128, with a dense size that is not a multiple of 32."""
    g = load_golden_layout("kat_4x3")
    run_case(mode, ta, tb, g["pattern"], 16, 40, dtype, "auto", batch=(3,), seed=77)
    run_case(mode, ta, tb, _wide_pattern(), 16, 64, dtype, "auto", batch=(1,), seed=78)
    run_case(mode, ta, tb, g["pattern"], 128, 64, dtype, "auto", batch=(1,), seed=79)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_block128_on_tensor_cores(mode, ta, tb, dtype):
    """Block 128 on the tcgen05 engine, requested explicitly (it must not fall back): every block is
    walked as 2 x 2 tiles of 64 x 64.  Non-square pattern with empty groups, several work items per
    CTA, dense sizes that leave a partial slice."""
    g = load_golden_layout("empty_row_col_5x4")
    run_case(mode, ta, tb, g["pattern"], 128, 64, dtype, "tcgen05", batch=(2,), seed=131)
    rng = np.random.default_rng(5)
    pattern = (rng.random((9, 7)) < 0.4).astype(np.int64)
    pattern[3, :] = 0
    run_case(mode, ta, tb, pattern, 128, 160, dtype, "tcgen05", batch=(5, 8), seed=132)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
@pytest.mark.parametrize("block", [64, 128])
def test_fp32_block64_and_block128_on_tensor_cores(mode, ta, tb, block):
    """fp32 at blocks 64 and 128 on the tcgen05 engine as a 3xTF32 split, requested explicitly (it must not
    fall back): every block is walked as 2 x 2 / 4 x 4 panels of 32 x 32.  Patterns with empty groups, several
    work items per CTA, dense sizes that leave partial slices; tolerance 1e-4 against the fp64 oracle."""
    g = load_golden_layout("empty_row_col_5x4")
    run_case(mode, ta, tb, g["pattern"], block, 64, torch.float32, "tcgen05", batch=(2,), seed=231)
    rng = np.random.default_rng(7)
    pattern = (rng.random((9, 7)) < 0.4).astype(np.int64)
    pattern[3, :] = 0
    run_case(mode, ta, tb, pattern, block, 96 if block == 64 else 160, torch.float32, "tcgen05", batch=(3, 4), seed=232)


def test_config1_sdd_fp32_per_head_layouts():
    """benchmark configuration 1: batch 1, heads 2, seq 256, head_dim 64, block 32, Bernoulli(0.5) + diagonal
    per head, Q.K^T as sdd(N,T) in fp32."""
    for head in range(2):
        g = load_golden_layout("cfg1_head%d" % head)
        q = seeded((1, 256, 64), 1000 + head)
        k = seeded((1, 256, 64), 1100 + head)
        from sparse import SparseLayout, matmul
        layout = SparseLayout(torch.tensor(g["pattern"]))
        got = matmul(q.cuda(), k.cuda(), "sdd", layout, False, True)
        ref = oracle.sparse_matmul(q, k, "sdd", np.array(g["pattern"]), 32, False, True, dtype=torch.float64)
        assert_close(got, ref, torch.float32, "config 1 head %d" % head)


@pytest.mark.parametrize("mode,ta,tb", VARIANTS)
def test_config4_fp32_stress_slice(mode, ta, tb):
    """benchmark configuration 4 on one head: seq 2048, head_dim 128, block 32, Bernoulli(0.1) + diagonal,
    inputs U(-1, 1), all modes and transpositions, fp32 tolerance 1e-4."""
    g = load_golden_layout("cfg4_head0")
    run_case(mode, ta, tb, g["pattern"], 32, 128, torch.float32, "auto", batch=(1,), seed=4000, dist="uniform")


@pytest.mark.parametrize("block,dim,seq,slices", [(64, 128, 8192, 512), (64, 64, 4096, 1024), (32, 64, 4096, 512)])
def test_sdd_with_thousands_of_accumulations_per_cta(block, dim, seq, slices):
    """sdd over many batch entries: every CTA runs through some thousand accumulations, so its two issue pipelines
    (even and odd accumulations) drift far apart.  The result must equal, bit for bit, the same slices computed
    32 at a time (short launches, the size the oracle comparisons cover), launch after launch, and no kernel may
    report a bounded wait that ran out.  (The largest case is benchmark configuration 5's Q.K^T.)"""
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    from sparse.patterns import bigbird
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(77)
    q, k = (torch.randn(slices, seq, dim, device="cuda", generator=gen).half() for _ in range(2))
    rl, cl = lay.row_layout, lay.col_layout
    parts = torch.cat([sparse_ops.sparse_matmul(q[i:i + 32], k[i:i + 32], "sdd", rl, cl, False, True, block)
                       for i in range(0, slices, 32)])
    sparse_ops.check_device_status(0)
    for launch in range(6):
        whole = sparse_ops.sparse_matmul(q, k, "sdd", rl, cl, False, True, block)
        sparse_ops.check_device_status(0)
        assert torch.equal(whole, parts), "launch %d differs from the 32-slice launches" % launch
        del whole


@pytest.mark.parametrize("mode,ta,tb", [("dsd", False, False), ("dsd", True, False), ("dds", False, False), ("dds", False, True)])
@pytest.mark.parametrize("block,dim,seq,slices", [(64, 128, 4096, 512), (32, 64, 4096, 512)])
def test_dsd_dds_with_hundreds_of_groups_per_cta(mode, ta, tb, block, dim, seq, slices):
    """The dense-output modes over 512 batch entries (every CTA walks several hundred block rows or columns,
    its stage and accumulator barriers wrap thousands of times): bit for bit the result of 32-slice launches,
    launch after launch, and no bounded wait runs out."""
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    from sparse.patterns import bigbird
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(78)
    sp = torch.randn(slices, lay.num_blocks, block, block, device="cuda", generator=gen).half()
    dn = torch.randn(slices, dim, seq, device="cuda", generator=gen).half() if mode == "dds" else \
        torch.randn(slices, seq, dim, device="cuda", generator=gen).half()
    a, b = (sp, dn) if mode == "dsd" else (dn, sp)
    rl, cl = lay.row_layout, lay.col_layout
    parts = torch.cat([sparse_ops.sparse_matmul(a[i:i + 32], b[i:i + 32], mode, rl, cl, ta, tb, block)
                       for i in range(0, slices, 32)])
    sparse_ops.check_device_status(0)
    for launch in range(4):
        whole = sparse_ops.sparse_matmul(a, b, mode, rl, cl, ta, tb, block)
        sparse_ops.check_device_status(0)
        assert torch.equal(whole, parts), "launch %d differs from the 32-slice launches" % launch
        del whole


@pytest.mark.parametrize("mode,ta,tb", [("sdd", False, True), ("dsd", False, False), ("dds", False, True)])
@pytest.mark.parametrize("block,dim,seq,slices,dtype", [
    (32, 128, 2048, 256, torch.float32),        # 3xTF32 through the block-32 engine (splitter warps in the pipeline)
    (64, 64, 2048, 256, torch.float32),         # 3xTF32 through the block-64 engine
    (128, 64, 4096, 256, torch.float16),        # blocks walked as 2 x 2 tiles
    (16, 64, 1024, 512, torch.float16),         # block 16
    (64, 64, 4096, 512, torch.bfloat16),
])
def test_long_launches_of_the_other_engines_and_types(mode, ta, tb, block, dim, seq, slices, dtype):
    """Hundreds of work items per CTA for the instances the 16-bit block-32 / block-64 cases above do not reach:
    the result of one launch over all slices must equal, bit for bit, 32-slice launches, and no bounded wait may
    run out."""
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    from sparse.patterns import bigbird
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(80)
    def rnd(*shape):
        return torch.randn(*shape, device="cuda", generator=gen).to(dtype)
    if mode == "sdd":
        a, b = rnd(slices, seq, dim), rnd(slices, seq, dim)
    elif mode == "dsd":
        a, b = rnd(slices, lay.num_blocks, block, block), rnd(slices, seq, dim)
    else:
        a, b = rnd(slices, dim, seq), rnd(slices, lay.num_blocks, block, block)
    rl, cl = lay.row_layout, lay.col_layout
    parts = torch.cat([sparse_ops.sparse_matmul(a[i:i + 32], b[i:i + 32], mode, rl, cl, ta, tb, block)
                       for i in range(0, slices, 32)])
    sparse_ops.check_device_status(0)
    for launch in range(3):
        whole = sparse_ops.sparse_matmul(a, b, mode, rl, cl, ta, tb, block)
        sparse_ops.check_device_status(0)
        assert torch.equal(whole, parts), "launch %d differs from the 32-slice launches" % launch
        del whole


def test_autograd_matches_dense_autograd():
    """Gradients through sparse.matmul equal those of the dense masked computation."""
    from sparse import SparseLayout, matmul
    g = load_golden_layout("kat_4x3")
    pattern = np.array(g["pattern"])
    block = 32
    layout = SparseLayout(torch.tensor(pattern), block=block)
    for mode, ta, tb in VARIANTS:
        a, b = operands(mode, ta, tb, pattern, block, 64, (2,), 21, torch.float32)
        ag, bg = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
        out = matmul(ag, bg, mode, layout, ta, tb)
        dc = seeded(tuple(out.shape), 23)
        out.backward(dc.cuda())
        ad, bd = a.double().requires_grad_(True), b.double().requires_grad_(True)
        a_full = oracle.to_dense(ad, pattern, block) if mode[1] == "s" else ad
        b_full = oracle.to_dense(bd, pattern, block) if mode[2] == "s" else bd
        c = (a_full.transpose(-1, -2) if ta else a_full) @ (b_full.transpose(-1, -2) if tb else b_full)
        if mode[0] == "s":
            c = oracle.to_sparse(c, pattern, block)
        c.backward(dc.double())
        assert_close(ag.grad, ad.grad, torch.float32, "dA %s %s %s" % (mode, ta, tb))
        assert_close(bg.grad, bd.grad, torch.float32, "dB %s %s %s" % (mode, ta, tb))


def test_argument_validation_raises():
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    layout = SparseLayout(torch.tensor([[1, 0], [1, 1]]))
    q = torch.randn(1, 64, 64, device="cuda")
    with pytest.raises(RuntimeError):
        sparse_ops.sparse_matmul(q, q, "ssd", layout.row_layout, layout.col_layout, False, True, 32, "auto")
    with pytest.raises(RuntimeError):
        sparse_ops.sparse_matmul(q, q.double(), "sdd", layout.row_layout, layout.col_layout, False, True, 32, "auto")
    with pytest.raises(RuntimeError):   # seq 96 does not match the 2-row layout
        sparse_ops.sparse_matmul(torch.randn(1, 96, 64, device="cuda"), q, "sdd", layout.row_layout,
                                 layout.col_layout, False, True, 32, "auto")
    with pytest.raises(RuntimeError):   # int tensors are rejected, not silently ignored
        sparse_ops.sparse_matmul(q.int(), q.int(), "sdd", layout.row_layout, layout.col_layout, False, True, 32,
                                 "auto")
    with pytest.raises(RuntimeError):   # wrong number of blocks in the sparse operand
        sparse_ops.sparse_matmul(torch.randn(1, 5, 32, 32, device="cuda"), q, "dsd", layout.row_layout,
                                 layout.col_layout, False, False, 32, "auto")


def test_dense_operand_shorter_than_the_layout_is_rejected():
    """The axis the chosen layout does not group is checked against the other layout: a dense operand that
    is shorter than the pattern would be read beyond its end by the blocks of the last columns / rows."""
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    layout = SparseLayout(torch.tensor([[1, 0, 1], [1, 1, 1]]), block=32)       # 2 x 3 blocks
    rl, cl = layout.row_layout, layout.col_layout
    nnz = layout.num_blocks
    p = torch.randn(1, nnz, 32, 32, device="cuda")
    for engine in ("auto", "simt"):
        with pytest.raises(RuntimeError):   # dsd: b needs 3 * 32 rows
            sparse_ops.sparse_matmul(p, torch.randn(1, 64, 64, device="cuda"), "dsd", rl, cl, False, False, 32, engine)
        with pytest.raises(RuntimeError):   # sdd: op(b) needs 3 * 32 columns
            sparse_ops.sparse_matmul(torch.randn(1, 64, 64, device="cuda"), torch.randn(1, 64, 64, device="cuda"),
                                     "sdd", rl, cl, False, True, 32, engine)
        with pytest.raises(RuntimeError):   # dds: a needs 2 * 32 columns
            sparse_ops.sparse_matmul(torch.randn(1, 64, 96, device="cuda"), p, "dds", rl, cl, False, False, 32, engine)
        ok = sparse_ops.sparse_matmul(p, torch.randn(1, 96, 64, device="cuda"), "dsd", rl, cl, False, False, 32, engine)
        assert ok.shape == (1, 64, 64)


@pytest.mark.skipif(not os.environ.get("BSA_REFERENCE_CHECKOUT"),
                    reason="set BSA_REFERENCE_CHECKOUT to a checkout of the reference project")
def test_reference_autograd_layer_unmodified_over_this_binding():
    """The reference's own sparse/matmul.py, imported unmodified from a checkout, with its `sparse_ops`
    replaced by the binding of this library (seven positional arguments, the reference call): gradients equal
    dense autograd for all twelve (mode, trans_a, trans_b) variants."""
    import importlib
    import types
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    root = os.environ["BSA_REFERENCE_CHECKOUT"]
    pkg = types.ModuleType("refsparse")
    pkg.__path__ = [os.path.join(root, "sparse")]
    sys.modules["refsparse"] = pkg
    kernel = types.ModuleType("refsparse.kernel")
    kernel.sparse_ops = sparse_ops                 # the reference calls sparse_ops.sparse_matmul(a, b, mode, rl, cl, ta, tb)
    sys.modules["refsparse.kernel"] = kernel
    ref_matmul = importlib.import_module("refsparse.matmul").matmul
    g = load_golden_layout("kat_4x3")
    pattern = np.array(g["pattern"])
    block = 32                                     # the reference's only block size (the binding's default)
    layout = SparseLayout(torch.tensor(pattern), block=block)
    for mode, ta, tb in VARIANTS:
        a, b = operands(mode, ta, tb, pattern, block, 64, (2,), 31, torch.float32)
        ag, bg = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
        out = ref_matmul(ag, bg, mode, layout, ta, tb)
        dc = seeded(tuple(out.shape), 33)
        out.backward(dc.cuda())
        ad, bd = a.double().requires_grad_(True), b.double().requires_grad_(True)
        a_full = oracle.to_dense(ad, pattern, block) if mode[1] == "s" else ad
        b_full = oracle.to_dense(bd, pattern, block) if mode[2] == "s" else bd
        c = (a_full.transpose(-1, -2) if ta else a_full) @ (b_full.transpose(-1, -2) if tb else b_full)
        if mode[0] == "s":
            c = oracle.to_sparse(c, pattern, block)
        c.backward(dc.double())
        assert_close(out, c, torch.float32, "C %s %s %s" % (mode, ta, tb))
        assert_close(ag.grad, ad.grad, torch.float32, "dA %s %s %s" % (mode, ta, tb))
        assert_close(bg.grad, bd.grad, torch.float32, "dB %s %s %s" % (mode, ta, tb))
