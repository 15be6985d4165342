"""GPU parity of the fused block-sparse attention backward kernels (dQ by block rows, dK and dV by
block columns) against dense masked attention differentiated by torch autograd on the CPU.
Tolerance: the 16-bit contract of the unfused operators (max |got - ref| / max |ref| <= 1e-2 for
fp16, 3e-2 for bf16)."""
import importlib

import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden_layout, seeded
from oracle import oracle

pytestmark = pytest.mark.gpu


def _grads(pattern, batch, dim, dtype, scale, causal=False, kpm=None, seed=0, block=64):
    """(dq, dk, dv) through sparse.attention (fused forward and backward) and through the oracle."""
    from sparse import SparseLayout, attention
    from sparse.kernel import sparse_ops
    pattern = torch.as_tensor(np.asarray(pattern))
    layout = SparseLayout(pattern, block=block)
    seq_q, seq_k = pattern.shape[0] * block, pattern.shape[1] * block
    q = seeded(tuple(batch) + (seq_q, dim), seed, dtype)
    k = seeded(tuple(batch) + (seq_k, dim), seed + 1, dtype)
    v = seeded(tuple(batch) + (seq_k, dim), seed + 2, dtype)
    do = seeded(tuple(batch) + (seq_q, dim), seed + 3, dtype)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = attention(qg, kg, vg, layout, scale, causal, None if kpm is None else kpm.cuda())
    out.backward(do.cuda())
    torch.cuda.synchronize()
    sparse_ops.check_device_status(0)
    ref, dq, dk, dv = oracle.attention_step_dense(q, k, v, do, pattern.numpy(), block, scale, causal,
                                                  key_padding_mask=kpm)
    assert_close(out, ref, dtype, "output")
    assert_close(qg.grad, dq, dtype, "dQ")
    assert_close(kg.grad, dk, dtype, "dK")
    assert_close(vg.grad, dv, dtype, "dV")
    return qg.grad, kg.grad, vg.grad, pattern


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_backward_strided_local(dim, dtype):
    from sparse.patterns import strided_local
    _grads(strided_local(16, 4, 1), (3,), dim, dtype, dim ** -0.5, seed=200)


@pytest.mark.parametrize("dim", [64, 128])
def test_backward_empty_rows_and_columns_nonsquare(dim):
    """An empty block row gives zero dQ rows, an empty block column zero dK / dV rows."""
    g = load_golden_layout("empty_row_col_5x4")
    dq, dk, dv, pattern = _grads(g["pattern"], (3,), dim, torch.float16, 0.2, seed=210)
    on = pattern != 0
    for r in range(pattern.shape[0]):
        if not bool(on[r].any()):
            assert float(dq[:, r * 64:(r + 1) * 64].abs().max()) == 0.0
    for c in range(pattern.shape[1]):
        if not bool(on[:, c].any()):
            assert float(dk[:, c * 64:(c + 1) * 64].abs().max()) == 0.0
            assert float(dv[:, c * 64:(c + 1) * 64].abs().max()) == 0.0


@pytest.mark.parametrize("dim", [64, 128])
def test_backward_causal_and_key_padding(dim):
    """Element-level causal mask on diagonal blocks, padded keys, and query rows left without any
    unmasked score (padding covers everything the causal mask leaves): their gradients are zero."""
    from sparse.patterns import local_global_causal
    kpm = torch.zeros(2, 512, dtype=torch.uint8)
    kpm[0, 300:] = 1
    kpm[1, :70] = 1            # rows 0 .. 69 of these batch entries see no key at all
    _grads(local_global_causal(8, 2, 1), (2, 3), dim, torch.float16, dim ** -0.5, True, kpm, seed=220)
    _grads(local_global_causal(8, 2, 1), (2,), dim, torch.bfloat16, dim ** -0.5, True, None, seed=221)


def test_backward_many_items_per_cta():
    """More work items than CTAs (8 heads x 64 block rows / columns), groups of 1 to 64 blocks."""
    from sparse.patterns import bigbird
    _grads(bigbird(64, 1, 2, 3, 77), (8,), 64, torch.float16, 0.125, seed=230)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_short_rows_and_several_items_per_cta(causal, dim):
    """Block rows and columns of 1 to 3 blocks with four to five work items per CTA, with and without the
    element-level masks: the hand-over of the accumulators between consecutive items happens after very
    few blocks, so every barrier involved must be waited on by the same warps in every phase (an earlier
    version let the owner of an item's last block finish the item and ran into a time-out here)."""
    from sparse.patterns import local_global_causal
    _grads(local_global_causal(16, 2, 1), (40,), dim, torch.float16, dim ** -0.5, causal, None, seed=260)


def test_backward_negative_scale():
    from sparse.patterns import strided_local
    _grads(strided_local(8, 4, 1), (2,), 64, torch.float16, -0.2, seed=240)


@pytest.mark.parametrize("dim", [64, 128])
def test_fused_backward_agrees_with_unfused_composition(dim):
    """Fused and unfused backward of the same fused forward agree far inside the tolerance."""
    from sparse import SparseLayout
    from sparse.patterns import strided_local
    module = importlib.import_module("sparse.attention")
    layout = SparseLayout(strided_local(64, 8, 2), block=64)
    q, k, v, do = (seeded((4, 4096, dim), 250 + i, torch.float16).cuda() for i in range(4))
    grads = {}
    try:
        for fused in (True, False):
            module.fused_backward = fused
            qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
            module.attention(qg, kg, vg, layout, dim ** -0.5).backward(do)
            grads[fused] = (qg.grad, kg.grad, vg.grad)
    finally:
        module.fused_backward = True
    for a, b, name in zip(grads[True], grads[False], ("dQ", "dK", "dV")):
        err = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert err <= 4e-3, (name, err)


@pytest.mark.parametrize("causal", [False, True])
def test_many_rows_per_pipeline_wrap_the_entry_rings(causal):
    """Seventeen or more block rows (and thirty or more block columns) per pipeline at head dim 64: the
    eight-entry rings through which a pipeline's producer hands rows, columns and block descriptors to its
    issuers and compute warps wrap several times.  Rows without blocks are mixed in (the producer zeroes them
    and the other roles never see them).  Fused forward and backward against the unfused composition."""
    from sparse import SparseLayout
    module = importlib.import_module("sparse.attention")
    rows = 32
    pattern = torch.zeros(rows, rows, dtype=torch.uint8)
    for i in range(rows):
        if i % 7 == 3:
            continue                                    # a row without blocks
        pattern[i, i] = 1
        pattern[i, (5 * i + 1) % rows if not causal else (i // 2)] = 1
    pattern[:, 11] = 0                                  # a column without blocks
    layout = SparseLayout(pattern, block=64)
    z = 330                                             # 10 560 rows over 592 row / 296 column pipelines
    q, k, v, do = (seeded((z, rows * 64, 64), 270 + i, torch.float16).cuda() for i in range(4))
    out, grads = {}, {}
    try:
        for fused in (True, False):
            module.fused_backward = fused
            qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
            if fused:
                o = module.attention(qg, kg, vg, layout, 0.125, causal)
            else:
                from sparse import matmul, softmax
                o = matmul(softmax(matmul(qg, kg, "sdd", layout, False, True), layout, scale=0.125, causal=causal), vg, "dsd", layout)
            o.backward(do)
            out[fused], grads[fused] = o.detach(), (qg.grad, kg.grad, vg.grad)
    finally:
        module.fused_backward = True
    sparse_kernel = importlib.import_module("sparse.kernel")
    sparse_kernel.sparse_ops.check_device_status(0)
    for a, b, name in zip((out[True],) + grads[True], (out[False],) + grads[False], ("O", "dQ", "dK", "dV")):
        err = float((a.float() - b.float()).abs().max() / b.float().abs().max())
        assert err <= 5e-3, (name, err)
        assert torch.isfinite(a.float()).all(), name


@pytest.mark.parametrize("block,dim,causal", [(64, 64, False), (64, 64, True), (64, 128, False), (32, 64, True)])
def test_fused_step_with_hundreds_of_rows_per_pipeline(block, dim, causal):
    """512 slices of seq 4096: every pipeline of the fused kernels walks more than a hundred block rows (columns)
    and its rings wrap throughout.  Output and gradients must equal, bit for bit, those of 32-slice launches
    (the size the oracle comparisons cover), launch after launch, and no bounded wait may run out."""
    from sparse import SparseLayout, attention
    from sparse.patterns import bigbird
    seq, slices = 4096, 512
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(79)
    q, k, v, do = (torch.randn(slices, seq, dim, device="cuda", generator=gen).half() for _ in range(4))

    def step(lo, hi):
        qg, kg, vg = (t[lo:hi].detach().clone().requires_grad_(True) for t in (q, k, v))
        o = attention(qg, kg, vg, lay, dim ** -0.5, causal)
        o.backward(do[lo:hi])
        return o.detach(), qg.grad, kg.grad, vg.grad

    sparse_kernel = importlib.import_module("sparse.kernel")
    parts = [torch.cat(t) for t in zip(*(step(i, i + 32) for i in range(0, slices, 32)))]
    sparse_kernel.sparse_ops.check_device_status(0)
    for launch in range(4):
        whole = step(0, slices)
        sparse_kernel.sparse_ops.check_device_status(0)
        for got, ref, name in zip(whole, parts, ("O", "dQ", "dK", "dV")):
            assert torch.equal(got, ref), "launch %d: %s differs from the 32-slice launches" % (launch, name)
        del whole


@pytest.mark.parametrize("block,dim,dtype", [(64, 64, torch.bfloat16), (64, 128, torch.bfloat16), (32, 128, torch.float16), (16, 64, torch.float16)])
def test_fused_step_long_launch_with_padding_mask(block, dim, dtype):
    """256 slices of seq 2048 with a key-padding mask (the masked instances of the three fused kernels, and the
    general backward at head dim 128): equal, bit for bit, to 32-slice launches; no bounded wait runs out."""
    from sparse import SparseLayout, attention
    from sparse.patterns import bigbird
    seq, slices = 2048, 256
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(81)
    q, k, v, do = (torch.randn(slices, seq, dim, device="cuda", generator=gen).to(dtype) for _ in range(4))
    kpm = torch.zeros(slices, seq, dtype=torch.uint8, device="cuda")
    kpm[:, seq - 100:] = 1
    kpm[1::3, 500:530] = 1

    def step(lo, hi):
        qg, kg, vg = (t[lo:hi].detach().clone().requires_grad_(True) for t in (q, k, v))
        o = attention(qg, kg, vg, lay, dim ** -0.5, False, kpm[lo:hi])
        o.backward(do[lo:hi])
        return o.detach(), qg.grad, kg.grad, vg.grad

    sparse_kernel = importlib.import_module("sparse.kernel")
    parts = [torch.cat(t) for t in zip(*(step(i, i + 32) for i in range(0, slices, 32)))]
    sparse_kernel.sparse_ops.check_device_status(0)
    for launch in range(3):
        whole = step(0, slices)
        sparse_kernel.sparse_ops.check_device_status(0)
        for got, ref, name in zip(whole, parts, ("O", "dQ", "dK", "dV")):
            assert torch.isfinite(got.float()).all(), name
            assert torch.equal(got, ref), "launch %d: %s differs from the 32-slice launches" % (launch, name)
        del whole


def test_full_size_fused_step_properties_config5():
    """Benchmark configuration 5 at full size (512 slices, seq 8192, head dim 128, BigBird layout) through
    the fused forward and backward, checked by size-independent properties: (1) with V = 1 every output
    element is 1 (probabilities sum to one); (2) then dQ = dK = 0 exactly up to rounding (dP = D_i in every
    row) and dV[j] = sum_i P_ij dO_i, whose sum over the keys of a slice equals the sum of dO over its
    queries; (3) the last slices of the full launch equal the same slices computed alone (an index overflow
    would hit the high slices)."""
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    from sparse.patterns import bigbird
    free, _ = torch.cuda.mem_get_info()
    if free < 24 * 2 ** 30:
        pytest.skip("needs about 16 GB of device memory")
    layout = SparseLayout(bigbird(128, 1, 2, 3, 5000), block=64)
    z, seq, d, scale = 512, 8192, 128, 128 ** -0.5
    rl, cl = layout.row_layout, layout.col_layout
    gen = torch.Generator(device="cuda").manual_seed(55)
    q = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    k = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    do = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    ones = torch.ones(z, seq, d, device="cuda", dtype=torch.float16)
    o, lse = sparse_ops.sparse_attention_forward(q, k, ones, rl[0], rl[1], 64, 128, scale, False, None)
    assert float((o.float() - 1).abs().max()) < 1e-2
    dq, dk, dv = sparse_ops.sparse_attention_backward(q, k, ones, o, do, lse, rl[0], rl[1], cl[0], cl[1], 64,
                                                      scale, False, None)
    sparse_ops.check_device_status(0)
    # dP - D_i = rowsum(dO) - sum_d dO o O with O = 1 +- rounding: tiny against |dO| ~ 1
    assert float(dq.float().abs().max()) < 5e-2 and float(dk.float().abs().max()) < 5e-2
    col_sums = dv[-4:].float().sum(dim=1)
    row_sums = do[-4:].float().sum(dim=1)
    assert float((col_sums - row_sums).abs().max() / row_sums.abs().max()) < 1e-2
    v = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    o, lse = sparse_ops.sparse_attention_forward(q, k, v, rl[0], rl[1], 64, 128, scale, False, None)
    dq, dk, dv = sparse_ops.sparse_attention_backward(q, k, v, o, do, lse, rl[0], rl[1], cl[0], cl[1], 64,
                                                      scale, False, None)
    tail = slice(z - 3, z)
    o2, lse2 = sparse_ops.sparse_attention_forward(q[tail], k[tail], v[tail], rl[0], rl[1], 64, 128, scale, False, None)
    dq2, dk2, dv2 = sparse_ops.sparse_attention_backward(q[tail], k[tail], v[tail], o2, do[tail], lse2, rl[0], rl[1],
                                                         cl[0], cl[1], 64, scale, False, None)
    sparse_ops.check_device_status(0)
    assert torch.equal(o[tail], o2) and torch.equal(lse[tail], lse2)
    assert torch.equal(dq[tail], dq2) and torch.equal(dk[tail], dk2) and torch.equal(dv[tail], dv2)


@pytest.mark.parametrize("dim,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_block32_layout_runs_fused_with_quadrant_masks(dim, dtype):
    """A layout of 32 x 32 blocks goes through the fused kernels as the layout of the 64 x 64 blocks that
    contain its blocks, with a 4-bit quadrant mask per block: forward and backward against dense autograd,
    on a random pattern (every combination of quadrants, coarse rows whose upper or lower half is empty)
    with padded keys, and on benchmark configuration 2's causal layout."""
    from sparse import SparseLayout
    from sparse.attention import _kernel_layout, fused_supported
    from sparse.patterns import local_global_causal
    rng = np.random.default_rng(32)
    pattern = (rng.random((12, 10)) < 0.3).astype(np.int64)
    pattern[5, :] = 0                     # an empty block row inside a coarse row
    pattern[:, 4] = 0
    layout = SparseLayout(torch.as_tensor(pattern), block=32)
    assert fused_supported(torch.empty(1, 1, dim, device="cuda", dtype=dtype), layout)
    assert _kernel_layout(layout).quadrant_masks
    kpm = torch.zeros(3, 320, dtype=torch.uint8)
    kpm[1, 200:] = 1
    kpm[2, :40] = 1
    _grads(pattern, (3, 2), dim, dtype, dim ** -0.5, False, kpm, seed=270, block=32)
    _grads(local_global_causal(32, 4, 1), (8,), dim, dtype, 0.125, True, None, seed=271, block=32)


def test_block32_with_odd_grid_composes_unfused_ops():
    from sparse import SparseLayout
    from sparse.attention import fused_supported
    g = load_golden_layout("empty_row_col_5x4")
    layout = SparseLayout(torch.as_tensor(np.asarray(g["pattern"])), block=32)
    assert not fused_supported(torch.empty(1, 1, 64, device="cuda", dtype=torch.float16), layout)
    _grads(g["pattern"], (2,), 64, torch.float16, 0.2, seed=272, block=32)
