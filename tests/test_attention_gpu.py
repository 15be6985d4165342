"""GPU parity of the whole block-sparse attention step (sdd -> softmax -> dsd, forward and
backward through autograd) on the benchmark configurations, against dense masked attention
on the CPU, plus size-independent properties at the full benchmark size."""
import numpy as np
import pytest
import torch

from conftest import assert_close, seeded

from oracle import oracle

pytestmark = pytest.mark.gpu


def sparse_attention(q, k, v, layout, scale, causal):
    from sparse import matmul, softmax
    s = matmul(q, k, "sdd", layout, False, True)
    p = softmax(s, layout, scale, causal)
    return matmul(p, v, "dsd", layout, False, False)


def _step(pattern, block, heads, seq, dim, dtype, scale, causal, seed, backward=True, dist="normal"):
    from sparse import SparseLayout
    layout = SparseLayout(pattern, block=block)
    q, k, v, do = (seeded((heads, seq, dim), seed + i, dtype, dist) for i in range(4))
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = sparse_attention(qg, kg, vg, layout, scale, causal)
    ref_out, dq, dk, dv = oracle.attention_step_dense(q, k, v, do if backward else None, pattern.numpy(), block,
                                                      scale, causal)
    assert_close(out, ref_out, dtype, "attention output")
    if backward:
        out.backward(do.cuda())
        assert_close(qg.grad, dq, dtype, "dQ")
        assert_close(kg.grad, dk, dtype, "dK")
        assert_close(vg.grad, dv, dtype, "dV")
    from sparse.kernel import sparse_ops
    sparse_ops.check_device_status(0)


def test_config2_causal_local_global_fp16():
    from sparse.patterns import local_global_causal
    _step(local_global_causal(32, 4, 1), 32, 3, 1024, 64, torch.float16, 0.125, True, 2000)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_block16_causal_step(dtype):
    """The smallest block size through the whole step (CUDA-core matmuls, softmax with 2 or 4 chunks per
    block row segment), forward and backward."""
    from sparse.patterns import local_global_causal
    _step(local_global_causal(16, 3, 1), 16, 3, 256, 64, dtype, 0.125, True, 2100)


def test_config3_strided_local_fp16_forward_backward():
    from sparse.patterns import strided_local
    _step(strided_local(64, 8, 2), 64, 2, 4096, 64, torch.float16, 0.125, False, 3000)


def test_config4_random_fp32_attention():
    from sparse.patterns import random_with_diagonal
    _step(random_with_diagonal(64, 64, 0.1, 4000), 32, 1, 2048, 128, torch.float32, 128 ** -0.5, False, 4000,
          dist="uniform")


def test_config5_bigbird_fp16_slice():
    from sparse.patterns import bigbird
    _step(bigbird(128, 1, 2, 3, 5000), 64, 1, 8192, 128, torch.float16, 128 ** -0.5, False, 5000)


def test_dds_formulation_of_dv_matches_dsd():
    """dV^T = dO^T . P computed as dds(T,N) equals the transpose of dV = P^T . dO computed as dsd(T,N)."""
    from sparse import SparseLayout, matmul
    from sparse.patterns import strided_local
    layout = SparseLayout(strided_local(64, 8, 2), block=64)
    p = torch.rand(2, layout.num_blocks, 64, 64, device="cuda").half()
    do = torch.randn(2, 4096, 64, device="cuda").half()
    dv = matmul(p, do, "dsd", layout, True, False)
    dvt = matmul(do, p, "dds", layout, True, False)
    assert_close(dvt.transpose(-1, -2), dv.float().cpu(), torch.float16, "dds vs dsd")


def test_full_size_properties_seq4096():
    """Benchmark workload (batch 4 x heads 16, seq 4096, d 64, block 64): properties that hold
    at any size.  (1) softmax rows sum to one: P . 1 = 1.  (2) sdd is linear in its first operand.
    (3) a head's result does not depend on which other heads share the launch."""
    from sparse import SparseLayout, matmul, softmax
    from sparse.patterns import strided_local
    layout = SparseLayout(strided_local(64, 8, 2), block=64)
    z, seq, d = 64, 4096, 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    q1 = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    q2 = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    k = torch.randn(z, seq, d, device="cuda", generator=gen).half()
    s1 = matmul(q1, k, "sdd", layout, False, True)
    p = softmax(s1, layout, 0.125)
    ones = torch.ones(z, seq, d, device="cuda", dtype=torch.float16)
    rowsum = matmul(p, ones, "dsd", layout, False, False)
    assert float((rowsum.float() - 1).abs().max()) < 1e-2
    s2 = matmul(q2, k, "sdd", layout, False, True)
    s12 = matmul((q1.float() + q2.float()).half(), k, "sdd", layout, False, True)
    lin = (s12.float() - (s1.float() + s2.float())).abs().max() / s12.float().abs().max()
    assert float(lin) < 1e-2
    sub = matmul(q1[5:7].contiguous(), k[5:7].contiguous(), "sdd", layout, False, True)
    assert torch.equal(sub, s1[5:7])
    from sparse.kernel import sparse_ops
    sparse_ops.check_device_status(0)


def test_full_size_config5_more_than_2_pow_31_elements():
    """benchmark configuration 5 at full size: batch 16 x heads 32 = 512 slices, seq 8192, head dim 128, block 64,
    BigBird layout with 1262 blocks: every sparse tensor has 2.65e9 elements (5.3 GB), beyond 32-bit
    element indices.  Checked through size-independent properties: (1) the last slices of the full
    launch equal the same slices computed alone (any index overflow would hit the high slices),
    (2) softmax rows sum to one, (3) the whole backward chain of the last slice equals the chain
    computed alone, (4) the fused forward agrees with the unfused one on the last slices."""
    from sparse import SparseLayout, matmul, softmax
    from sparse.attention import attention_lse
    from sparse.kernel import sparse_ops
    from sparse.patterns import bigbird
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2 ** 30:
        pytest.skip("needs about 30 GB of device memory")
    layout = SparseLayout(bigbird(128, 1, 2, 3, 5000), block=64)
    z, seq, d, scale = 512, 8192, 128, 128 ** -0.5
    assert z * layout.num_blocks * 64 * 64 > 2 ** 31
    gen = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, do = (torch.randn(z, seq, d, device="cuda", generator=gen).half() for _ in range(4))
    tail = slice(z - 3, z)

    def chain(q, k, v, do):
        s = matmul(q, k, "sdd", layout, False, True)
        p = softmax(s, layout, scale)
        del s
        o = matmul(p, v, "dsd", layout, False, False)
        dv = matmul(p, do, "dsd", layout, True, False)
        dp = matmul(do, v, "sdd", layout, False, True)
        ds = sparse_ops.sparse_softmax_backward(p, dp, layout.row_layout[0], layout.row_layout[1], scale,
                                                layout.max_row_blocks)
        del dp
        dq = matmul(ds, k, "dsd", layout, False, False)
        dk = matmul(ds, q, "dsd", layout, True, False)
        return p, o, dv, ds, dq, dk

    full = chain(q, k, v, do)
    part = chain(q[tail].contiguous(), k[tail].contiguous(), v[tail].contiguous(), do[tail].contiguous())
    names = ["p", "o", "dv", "ds", "dq", "dk"]
    for name, a, b in zip(names, full, part):
        assert torch.equal(a[tail], b), "%s of the last slices differs between the full and the 3-slice launch" % name
    p_tail = full[0][tail]
    ones = torch.ones(3, seq, d, device="cuda", dtype=torch.float16)
    rowsum = matmul(p_tail.contiguous(), ones, "dsd", layout, False, False)
    assert float((rowsum.float() - 1).abs().max()) < 1e-2
    o_unfused_tail = full[1][tail].float()
    del full, part
    fused, lse = attention_lse(q, k, v, layout, scale)
    err = float((fused[tail].float() - o_unfused_tail).abs().max() / o_unfused_tail.abs().max())
    assert err <= 5e-3, err
    assert bool(torch.isfinite(lse).all())
    sparse_ops.check_device_status(0)
