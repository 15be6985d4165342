"""Seeded random sweeps on the GPU: many small layouts, batch sizes and flags, each comparing two
independent implementations of the same result (no CPU oracle in the loop, so a case costs
milliseconds).  The sweeps exist for the hand-over protocols of the persistent kernels: how many
items a CTA walks, how many blocks an item has, which warp group finishes it and whether the masked
or the plain code path runs all change the interleaving of the mbarrier phases.

* fused attention forward / backward against the composition of the unfused operators;
* the tensor-core matmul engines against the CUDA-core engine.

Tolerances: 16-bit results of two different summation orders, max |a - b| / max |b| <= 1e-2 (bf16 3e-2).
"""
import importlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    scale = float(b.float().abs().max())
    return float((a.float() - b.float()).abs().max()) / max(scale, 1e-6)


def _random_pattern(rng, rows, cols, density):
    pattern = (rng.random((rows, cols)) < density).astype(np.int64)
    if rng.random() < 0.5:
        pattern[rng.integers(rows), :] = 0          # an empty block row
    if rng.random() < 0.5:
        pattern[:, rng.integers(cols)] = 0          # an empty block column
    if rng.random() < 0.3:
        pattern[rng.integers(rows), :] = 1          # a full block row
    if pattern.sum() == 0:
        pattern[0, 0] = 1
    return pattern


@pytest.mark.parametrize("seed", range(12))
def test_fused_attention_against_unfused_composition(seed):
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    module = importlib.import_module("sparse.attention")
    rng = np.random.default_rng(1000 + seed)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for case in range(8):
        block = int(rng.choice([32, 64, 64, 128]))
        square = rng.random() < 0.6
        rows = int(rng.integers(1, 13)) * (2 if block == 32 else 1)
        cols = rows if square else int(rng.integers(1, 13)) * (2 if block == 32 else 1)
        if block == 128:
            rows, cols = min(rows, 6), min(cols, 6)
        pattern = _random_pattern(rng, rows, cols, float(rng.choice([0.15, 0.4, 0.8])))
        dim = int(rng.choice([64, 128]))
        dtype = torch.float16 if rng.random() < 0.7 else torch.bfloat16
        z = int(rng.choice([1, 3, 17, 40]))
        if rows * cols * block * block * z > 3e8:
            z = 3
        causal = bool(square and rng.random() < 0.5)
        kpm = None
        if rng.random() < 0.4:
            kpm = (torch.rand(z, cols * block, device="cuda", generator=gen) < 0.2).to(torch.uint8)
        scale = float(dim) ** -0.5
        layout = SparseLayout(torch.as_tensor(pattern), block=block)
        q = torch.randn(z, rows * block, dim, device="cuda", generator=gen).to(dtype)
        k = torch.randn(z, cols * block, dim, device="cuda", generator=gen).to(dtype)
        v = torch.randn(z, cols * block, dim, device="cuda", generator=gen).to(dtype)
        do = torch.randn(z, rows * block, dim, device="cuda", generator=gen).to(dtype)
        assert module.fused_supported(q, layout)
        results = {}
        for fused in (True, False):
            qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
            if fused:
                out = module.attention(qg, kg, vg, layout, scale, causal, kpm)
            else:
                from sparse import matmul, softmax
                s = matmul(qg, kg, "sdd", layout, False, True)
                out = matmul(softmax(s, layout, scale, causal, kpm), vg, "dsd", layout)
            out.backward(do)
            results[fused] = (out.detach(), qg.grad, kg.grad, vg.grad)
        torch.cuda.synchronize()
        sparse_ops.check_device_status(0)
        tol = 1e-2 if dtype == torch.float16 else 3e-2
        what = "seed %d case %d: block %d grid %dx%d z %d dim %d %s causal %s kpm %s" % (
            seed, case, block, rows, cols, z, dim, dtype, causal, kpm is not None)
        for name, a, b in zip(("out", "dq", "dk", "dv"), results[True], results[False]):
            assert torch.isfinite(a.float()).all(), (what, name)
            assert _rel(a, b) <= tol, (what, name, _rel(a, b))


@pytest.mark.parametrize("seed", range(8))
def test_tensor_core_engines_against_cuda_core_engine(seed):
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    rng = np.random.default_rng(2000 + seed)
    gen = torch.Generator(device="cuda").manual_seed(100 + seed)
    for case in range(10):
        block = int(rng.choice([32, 64, 128]))
        rows, cols = int(rng.integers(1, 10)), int(rng.integers(1, 10))
        pattern = _random_pattern(rng, rows, cols, float(rng.choice([0.2, 0.5, 0.9])))
        dtype = [torch.float16, torch.bfloat16, torch.float32][int(rng.integers(3))]
        if dtype == torch.float32 and block != 32:
            dtype = torch.float16                     # fp32 runs on tensor cores at block 32 only
        inner = int(rng.choice([64, 72, 128, 200]))
        z = int(rng.choice([1, 5, 33]))
        mode = str(rng.choice(["sdd", "dsd", "dds"]))
        ta, tb = bool(rng.integers(2)), bool(rng.integers(2))
        layout = SparseLayout(torch.as_tensor(pattern), block=block)
        nnz, m_sp, n_sp = layout.num_blocks, rows * block, cols * block

        def dense(r, c, transposed):
            shape = (z, c, r) if transposed else (z, r, c)
            return torch.randn(*shape, device="cuda", generator=gen).to(dtype)

        sparse = torch.randn(z, nnz, block, block, device="cuda", generator=gen).to(dtype)
        if mode == "sdd":
            a, b = dense(m_sp, inner, ta), dense(inner, n_sp, tb)
        elif mode == "dsd":
            a = sparse
            b = dense(m_sp if ta else n_sp, inner, tb)
        else:
            a = dense(inner, n_sp if tb else m_sp, ta)
            b = sparse
        got = {}
        for engine in ("tcgen05", "simt"):
            got[engine] = sparse_ops.sparse_matmul(a, b, mode, layout.row_layout, layout.col_layout, ta, tb, block, engine)
        torch.cuda.synchronize()
        sparse_ops.check_device_status(0)
        tol = {torch.float16: 1e-2, torch.bfloat16: 3e-2, torch.float32: 1e-4}[dtype]
        what = "seed %d case %d: %s ta %s tb %s block %d grid %dx%d inner %d z %d %s" % (
            seed, case, mode, ta, tb, block, rows, cols, inner, z, dtype)
        assert got["tcgen05"].shape == got["simt"].shape, what
        assert _rel(got["tcgen05"], got["simt"]) <= tol, (what, _rel(got["tcgen05"], got["simt"]))


@pytest.mark.parametrize("seed", range(6))
def test_one_launch_over_many_slices_equals_32_slice_launches(seed):
    """Random layouts with 64 to 2048 batch entries, so that every CTA walks up to a few hundred work items and
    its rings and barriers wrap throughout: one launch over all slices must equal 32-slice launches bit for bit
    (matmul of every mode and transposition, and the fused forward + backward), twice in a row, and no kernel
    may report a bounded wait that ran out."""
    from sparse import SparseLayout, attention
    from sparse.kernel import sparse_ops
    rng = np.random.default_rng(7000 + seed)
    gen = torch.Generator(device="cuda").manual_seed(300 + seed)
    for case in range(24):
        block = int(rng.choice([32, 64, 64, 128]))
        rows = int(rng.integers(2, 25)) * (2 if block == 32 else 1)
        if block == 128:
            rows = min(rows, 8)
        pattern = _random_pattern(rng, rows, rows, float(rng.choice([0.1, 0.3, 0.7])))
        dim = int(rng.choice([64, 128]))
        dtype = torch.float16 if rng.random() < 0.7 else torch.bfloat16
        seq = rows * block
        slices = int(rng.choice([256, 512, 1024, 2048]))
        while slices * seq * dim > 3e8 or slices * int(pattern.sum()) * block * block > 8e8:
            slices //= 2
        slices = max(64, slices // 32 * 32)
        lay = SparseLayout(torch.as_tensor(pattern), block=block, device="cuda")
        rl, cl = lay.row_layout, lay.col_layout

        def rnd(*shape):
            return torch.randn(*shape, device="cuda", generator=gen).to(dtype)

        kind = int(rng.integers(0, 4))
        what = "seed %d case %d: kind %d block %d grid %d dim %d %s slices %d" % (seed, case, kind, block, rows, dim, dtype, slices)
        if kind == 3:
            causal = bool(rng.random() < 0.5)
            q, k, v, do = (rnd(slices, seq, dim) for _ in range(4))

            def step(lo, hi):
                qg, kg, vg = (x[lo:hi].detach().clone().requires_grad_(True) for x in (q, k, v))
                o = attention(qg, kg, vg, lay, dim ** -0.5, causal)
                o.backward(do[lo:hi])
                return o.detach(), qg.grad, kg.grad, vg.grad

            parts = [torch.cat(x) for x in zip(*(step(i, i + 32) for i in range(0, slices, 32)))]
            for _ in range(2):
                whole = step(0, slices)
                sparse_ops.check_device_status(0)
                for a, b, name in zip(whole, parts, ("O", "dQ", "dK", "dV")):
                    assert torch.equal(a, b), (what, name)
        else:
            mode = ("sdd", "dsd", "dds")[kind]
            ta, tb = bool(rng.random() < 0.5), bool(rng.random() < 0.5)
            if mode == "sdd":
                a = rnd(slices, dim, seq) if ta else rnd(slices, seq, dim)
                b = rnd(slices, seq, dim) if tb else rnd(slices, dim, seq)
            elif mode == "dsd":
                a, b = rnd(slices, lay.num_blocks, block, block), (rnd(slices, dim, seq) if tb else rnd(slices, seq, dim))
            else:
                a, b = (rnd(slices, seq, dim) if ta else rnd(slices, dim, seq)), rnd(slices, lay.num_blocks, block, block)

            def run(lo, hi):
                return sparse_ops.sparse_matmul(a[lo:hi], b[lo:hi], mode, rl, cl, ta, tb, block)

            parts = torch.cat([run(i, i + 32) for i in range(0, slices, 32)])
            for _ in range(2):
                whole = run(0, slices)
                sparse_ops.check_device_status(0)
                assert torch.equal(whole, parts), what
