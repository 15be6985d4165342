"""One pattern per head in one launch (BatchedSparseLayout): every head's result must equal the
single-layout computation of that head against the dense masked CPU oracle.  Tolerances as for the
single-layout operators (fp32 1e-4, fp16 1e-2)."""
import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden_layout, seeded
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_config1_two_heads_with_their_own_layouts_in_one_launch():
    """Benchmark configuration 1: batch 1, heads 2, seq 256, head dim 64, block 32, a seeded Bernoulli(0.5)
    layout with forced diagonal per head; Q.K^T as one sdd launch over both heads, fp32."""
    from sparse import BatchedSparseLayout, batched_matmul
    patterns = torch.tensor([load_golden_layout("cfg1_head%d" % h)["pattern"] for h in range(2)])
    layout = BatchedSparseLayout(patterns, block=32)
    q = seeded((1, 2, 256, 64), 1000)
    k = seeded((1, 2, 256, 64), 1100)
    s = batched_matmul(q.cuda(), k.cuda(), "sdd", layout, False, True)
    assert s.shape == (1, layout.num_blocks, 32, 32)
    for h in range(2):
        ref = oracle.sparse_matmul(q[:, h], k[:, h], "sdd", patterns[h].numpy(), 32, False, True, dtype=torch.float64)
        assert_close(layout.head_blocks(s, h), ref, torch.float32, "head %d" % h)


@pytest.mark.parametrize("dtype,block,dim", [(torch.float32, 32, 128), (torch.float16, 64, 64)])
def test_per_head_random_layouts_attention_chain(dtype, block, dim):
    """Benchmark configuration 4 in small: a seeded Bernoulli(0.1) layout with forced diagonal per head,
    U(-1, 1) inputs, sdd -> softmax -> dsd over all heads at once, plus the two transposed products of
    the backward pass."""
    from sparse import BatchedSparseLayout, batched_matmul, batched_softmax
    from sparse.patterns import random_with_diagonal
    heads, grid = 5, 12
    patterns = torch.stack([random_with_diagonal(grid, grid, 0.15, 4000 + h) for h in range(heads)])
    layout = BatchedSparseLayout(patterns, block=block)
    seq = grid * block
    q, k, v, do = (seeded((2, heads, seq, dim), 4100 + i, dtype, "uniform") for i in range(4))
    scale = dim ** -0.5
    s = batched_matmul(q.cuda(), k.cuda(), "sdd", layout, False, True)
    p = batched_softmax(s, layout, scale)
    o = batched_matmul(p, v.cuda(), "dsd", layout, False, False)
    dv = batched_matmul(p, do.cuda(), "dsd", layout, True, False)
    assert o.shape == (2, heads, seq, dim) and dv.shape == (2, heads, seq, dim)
    for h in range(heads):
        pat = patterns[h].numpy()
        ref_s = oracle.sparse_matmul(q[:, h], k[:, h], "sdd", pat, block, False, True)
        ref_p = oracle.softmax_forward(ref_s, pat, block, scale)
        ref_o = oracle.sparse_matmul(ref_p, v[:, h], "dsd", pat, block, False, False)
        ref_dv = oracle.sparse_matmul(ref_p, do[:, h], "dsd", pat, block, True, False)
        assert_close(layout.head_blocks(p, h), ref_p, dtype, "P head %d" % h)
        assert_close(o[:, h], ref_o, dtype, "O head %d" % h)
        assert_close(dv[:, h], ref_dv, dtype, "dV head %d" % h)


def test_per_head_layouts_fused_attention_causal_with_padding():
    """Fused attention over heads with different causal patterns, a key-padding mask and gradients."""
    from sparse import BatchedSparseLayout, batched_attention
    from sparse.patterns import local_global_causal
    patterns = torch.stack([local_global_causal(8, 2, 1), local_global_causal(8, 4, 0), local_global_causal(8, 1, 2)])
    layout = BatchedSparseLayout(patterns, block=64)
    q, k, v, do = (seeded((2, 3, 512, 64), 4200 + i, torch.float16) for i in range(4))
    kpm = torch.zeros(2, 512, dtype=torch.uint8)
    kpm[0, 300:] = 1
    kpm[1, 7] = 1
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = batched_attention(qg, kg, vg, layout, 0.125, True, kpm.cuda())
    out.backward(do.cuda())
    for h in range(3):
        pat = patterns[h].numpy()
        qr, kr, vr = (t[:, h].float().requires_grad_(True) for t in (q, k, v))
        keep = oracle._score_mask(pat, 64, True, kpm, (2,))
        scores = ((qr @ kr.transpose(-1, -2)) * 0.125).masked_fill(~keep, float("-inf"))
        probs = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
        ref = probs @ vr
        ref.backward(do[:, h].float())
        assert_close(out[:, h], ref.detach(), torch.float16, "output head %d" % h)
        assert_close(qg.grad[:, h], qr.grad, torch.float16, "dQ head %d" % h)
        assert_close(kg.grad[:, h], kr.grad, torch.float16, "dK head %d" % h)
        assert_close(vg.grad[:, h], vr.grad, torch.float16, "dV head %d" % h)
