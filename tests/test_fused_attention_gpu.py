"""GPU parity of the fused block-sparse attention kernel (one launch for sdd -> softmax -> dsd)
against dense masked attention on the CPU.  Tolerance: the 16-bit contract of the unfused
operators (max |got - ref| / max |ref| <= 1e-2 for fp16, 3e-2 for bf16); the log-sum-exp is an
fp32 output and is compared absolutely (1e-3)."""
import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden_layout, seeded
from oracle import oracle

pytestmark = pytest.mark.gpu


def _forward_case(pattern, block, batch, dim, dtype, scale, causal=False, kpm=None, seed=0):
    from sparse import SparseLayout
    from sparse.attention import attention_lse
    from sparse.kernel import sparse_ops
    pattern = torch.as_tensor(np.asarray(pattern))
    layout = SparseLayout(pattern, block=block)
    seq_q, seq_k = pattern.shape[0] * block, pattern.shape[1] * block
    q = seeded(tuple(batch) + (seq_q, dim), seed, dtype)
    k = seeded(tuple(batch) + (seq_k, dim), seed + 1, dtype)
    v = seeded(tuple(batch) + (seq_k, dim), seed + 2, dtype)
    out, lse = attention_lse(q.cuda(), k.cuda(), v.cuda(), layout, scale, causal,
                             None if kpm is None else kpm.cuda())
    torch.cuda.synchronize()
    sparse_ops.check_device_status(0)
    ref, ref_lse = oracle.attention_forward_dense(q, k, v, pattern.numpy(), block, scale, causal, kpm)
    assert out.dtype == dtype and tuple(out.shape) == tuple(ref.shape)
    assert_close(out, ref, dtype, "fused attention output")
    lse = lse.float().cpu()
    dead = torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(lse), dead), "rows without an unmasked score must report lse = -inf"
    if (~dead).any():
        assert float((lse[~dead] - ref_lse[~dead]).abs().max()) <= 1e-3
    if dead.any():
        assert float(out.float().cpu()[dead].abs().max()) == 0.0
    return out


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_forward_strided_local(dim, dtype):
    from sparse.patterns import strided_local
    _forward_case(strided_local(64, 8, 2), 64, (2,), dim, dtype, dim ** -0.5, seed=10)


@pytest.mark.parametrize("dim", [64, 128])
def test_fused_forward_empty_rows_nonsquare(dim):
    g = load_golden_layout("empty_row_col_5x4")     # an empty block row: zeros and lse = -inf
    _forward_case(g["pattern"], 64, (3,), dim, torch.float16, 0.2, seed=20)


def test_fused_forward_many_items_per_cta():
    """More work items than resident CTAs (8 heads x 64 block rows = 512 items): every CTA walks
    several items, including rows of 1 block and of 64 blocks (BigBird-style global rows)."""
    from sparse.patterns import bigbird
    _forward_case(bigbird(64, 1, 2, 3, 77), 64, (8,), 64, torch.float16, 0.125, seed=30)


def test_fused_forward_causal_and_key_padding():
    from sparse.patterns import local_global_causal
    pattern = local_global_causal(16, 3, 1)
    _forward_case(pattern, 64, (2, 2), 64, torch.float16, 0.125, causal=True, seed=40)
    kpm = torch.zeros(2, 16 * 64, dtype=torch.uint8)
    kpm[0, 700:] = 1          # pads the tail of batch entry 0, so some rows lose whole blocks
    kpm[1, 5] = 1
    kpm[1, 64:128] = 1        # a whole block column padded
    _forward_case(pattern, 64, (2, 2), 128, torch.bfloat16, 0.1, causal=True, kpm=kpm, seed=41)
    full = np.ones((4, 4), dtype=np.int64)
    dead = torch.zeros(1, 256, dtype=torch.uint8)
    dead[0, :] = 1            # every key padded: all rows dead
    _forward_case(full, 64, (1,), 64, torch.float16, 1.0, kpm=dead, seed=42)


def test_fused_forward_zero_scale_with_masks():
    """Scale 0: every unmasked score counts the same (uniform attention) and masked ones stay excluded
    (the kernel marks them with infinities, which a zero factor must not turn into NaN)."""
    from sparse.patterns import local_global_causal
    kpm = torch.zeros(2, 512, dtype=torch.uint8)
    kpm[0, 100:140] = 1
    kpm[1, :70] = 1
    _forward_case(local_global_causal(8, 2, 1), 64, (2, 2), 64, torch.float16, 0.0, True, kpm, seed=45)


def test_fused_forward_negative_scale_and_large_scores():
    """The row maximum is taken after scaling (a negative scale flips it), and scores of a few
    hundred do not overflow the exponentials."""
    from sparse.patterns import strided_local
    _forward_case(strided_local(8, 4, 1), 64, (2,), 64, torch.float16, -0.3, seed=50)
    _forward_case(strided_local(8, 4, 1), 64, (2,), 64, torch.float16, 6.0, seed=51)


def test_fused_forward_running_maximum_is_raised_block_after_block():
    """Keys grow from block to block, so every block's scores exceed the running row maximum by far
    more than the slack the kernel tolerates: the accumulated output is rescaled at every block.
    A second case has the largest scores in the first block (never rescaled)."""
    from sparse import SparseLayout
    from sparse.attention import attention_lse
    from sparse.patterns import strided_local
    pattern = strided_local(16, 4, 2)
    layout = SparseLayout(pattern, block=64)
    for dim in (64, 128):
        for growth in (1.0, -1.0):
            q = seeded((3, 1024, dim), 90, torch.float16)
            k = seeded((3, 1024, dim), 91, torch.float16)
            v = seeded((3, 1024, dim), 92, torch.float16)
            ramp = torch.exp2(growth * torch.arange(16, dtype=torch.float32) / 3).repeat_interleave(64)   # up to 32x
            k = (k.float() * ramp[None, :, None] * (1.0 if growth > 0 else 32.0)).half()
            q = q.abs()          # same sign: the scores of a block scale with its keys
            k = k.abs()
            out, lse = attention_lse(q.cuda(), k.cuda(), v.cuda(), layout, 0.5)
            ref, ref_lse = oracle.attention_forward_dense(q, k, v, pattern.numpy(), 64, 0.5)
            assert_close(out, ref, torch.float16, "rescaled output dim %d growth %g" % (dim, growth))
            assert float((lse.float().cpu() - ref_lse).abs().max() / ref_lse.abs().max()) <= 1e-3


def test_fused_agrees_with_unfused_composition():
    """The fused kernel and the three unfused kernels agree far inside the tolerance."""
    from sparse import SparseLayout, matmul, softmax
    from sparse.attention import attention_lse
    from sparse.patterns import strided_local
    layout = SparseLayout(strided_local(64, 8, 2), block=64)
    q, k, v = (seeded((4, 4096, 64), 60 + i, torch.float16).cuda() for i in range(3))
    fused, _ = attention_lse(q, k, v, layout, 0.125)
    p = softmax(matmul(q, k, "sdd", layout, False, True), layout, 0.125)
    unfused = matmul(p, v, "dsd", layout, False, False)
    err = float((fused.float() - unfused.float()).abs().max() / unfused.float().abs().max())
    assert err <= 3e-3, err


def test_autograd_through_fused_attention():
    from sparse import SparseLayout, attention
    from sparse.patterns import strided_local
    pattern = strided_local(16, 4, 1)
    layout = SparseLayout(pattern, block=64)
    q, k, v, do = (seeded((2, 1024, 64), 70 + i, torch.float16) for i in range(4))
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = attention(qg, kg, vg, layout, 0.125)
    out.backward(do.cuda())
    ref, dq, dk, dv = oracle.attention_step_dense(q, k, v, do, pattern.numpy(), 64, 0.125, False)
    assert_close(out, ref, torch.float16, "output")
    assert_close(qg.grad, dq, torch.float16, "dQ")
    assert_close(kg.grad, dk, torch.float16, "dK")
    assert_close(vg.grad, dv, torch.float16, "dV")


@pytest.mark.parametrize("dim", [64, 128])
def test_fused_forward_block128_runs_as_split_block64_layout(dim):
    """A block-128 layout goes through the same kernel as the block-64 layout with every block
    split in 2 x 2; causal and key-padding masks are element-level and unchanged."""
    from sparse.patterns import local_global_causal
    g = load_golden_layout("empty_row_col_5x4")
    _forward_case(g["pattern"], 128, (2,), dim, torch.float16, 0.2, seed=90)
    kpm = torch.zeros(2, 8 * 128, dtype=torch.uint8)
    kpm[0, 700:] = 1
    kpm[1, :130] = 1
    _forward_case(local_global_causal(8, 2, 1), 128, (2, 3), dim, torch.bfloat16, dim ** -0.5, True, kpm, seed=91)


def test_autograd_through_fused_attention_block128():
    from sparse import SparseLayout, attention
    from sparse.patterns import local_global_causal
    pattern = local_global_causal(4, 2, 1)
    layout = SparseLayout(pattern, block=128)
    q, k, v, do = (seeded((2, 512, 64), 95 + i, torch.float16) for i in range(4))
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = attention(qg, kg, vg, layout, 0.125, True)
    out.backward(do.cuda())
    ref, dq, dk, dv = oracle.attention_step_dense(q, k, v, do, pattern.numpy(), 128, 0.125, True)
    assert_close(out, ref, torch.float16, "output")
    assert_close(qg.grad, dq, torch.float16, "dQ")
    assert_close(kg.grad, dk, torch.float16, "dK")
    assert_close(vg.grad, dv, torch.float16, "dV")


def test_attention_composes_unfused_ops_where_the_fused_kernel_does_not_apply():
    from sparse import SparseLayout, attention
    from sparse.patterns import local_global_causal
    pattern = local_global_causal(8, 2, 1)
    layout = SparseLayout(pattern, block=32)
    q, k, v = (seeded((2, 256, 64), 80 + i) for i in range(3))
    out = attention(q.cuda(), k.cuda(), v.cuda(), layout, 0.125, True)
    ref, _ = oracle.attention_forward_dense(q, k, v, pattern.numpy(), 32, 0.125, True)
    assert_close(out, ref, torch.float32, "fp32 block-32 attention")


def test_self_attention_module_matches_dense_reference():
    """The nn.Module (QKV projection -> block-sparse attention -> output projection) against the same
    computation with dense masked attention, forward and the gradient of the input."""
    from sparse import SparseLayout, BlockSparseSelfAttention
    from sparse.patterns import local_global_causal
    pattern = local_global_causal(8, 3, 1)
    layout = SparseLayout(pattern, block=64)
    torch.manual_seed(0)
    mod = BlockSparseSelfAttention(256, 4, layout, causal=True, device="cuda", dtype=torch.float16)
    x = (0.5 * seeded((2, 512, 256), 95, torch.float16)).cuda().requires_grad_(True)
    y = mod(x)
    y.float().square().mean().backward()
    # dense reference with the same weights, in fp32 on the CPU
    xr = x.detach().float().cpu().requires_grad_(True)
    w_qkv, b_qkv = mod.qkv.weight.detach().float().cpu(), mod.qkv.bias.detach().float().cpu()
    w_out, b_out = mod.out.weight.detach().float().cpu(), mod.out.bias.detach().float().cpu()
    qkv = (xr @ w_qkv.t() + b_qkv).view(2, 512, 3, 4, 64).permute(2, 0, 3, 1, 4)
    keep = oracle._score_mask(pattern.numpy(), 64, True, None, (2, 4))
    scores = (qkv[0] @ qkv[1].transpose(-1, -2)) * 64 ** -0.5
    probs = torch.softmax(scores.masked_fill(~keep, float("-inf")), dim=-1)
    ref = (probs @ qkv[2]).transpose(1, 2).reshape(2, 512, 256) @ w_out.t() + b_out
    ref.square().mean().backward()
    assert_close(y, ref.detach(), torch.float16, "module output")
    # the gradient runs through six fp16 GEMMs and the softmax backward: three times the single-operator tolerance
    g, gr = x.grad.float().cpu(), xr.grad
    assert float((g - gr).abs().max() / gr.abs().max()) <= 3e-2


@pytest.mark.gpu
def test_debug_checks_run_after_forward_and_backward():
    """With `sparse.kernel.debug_checks` set every autograd op reads the device status after its forward and
    its backward pass; on a healthy run nothing is raised and the results are unchanged."""
    import importlib
    from sparse import SparseLayout, attention, matmul, softmax
    from sparse.patterns import strided_local
    kernel = importlib.import_module("sparse.kernel")
    layout = SparseLayout(strided_local(8, 4, 1), block=64)
    q, k, v = (seeded((2, 512, 64), 700 + i, torch.float16).cuda().requires_grad_(True) for i in range(3))
    ref = attention(q, k, v, layout, 0.125)
    old = kernel.debug_checks
    try:
        kernel.debug_checks = True
        out = attention(q, k, v, layout, 0.125)
        out.float().sum().backward()
        probs = softmax(matmul(q, k, "sdd", layout, False, True), layout, scale=0.125)
        matmul(probs, v, "dsd", layout).float().sum().backward()
    finally:
        kernel.debug_checks = old
    assert torch.equal(out, ref)
