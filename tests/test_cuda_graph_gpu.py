"""The operators under CUDA graph capture: a whole attention step (forward and backward) captured once with
torch.cuda.graphs and replayed must reproduce the eager results bit for bit.  What capture needs from the
library: every launch goes to the caller's stream, no entry point synchronises or allocates behind torch's
back, and the tensor maps are passed by value with the launch.  Small steps (benchmark configuration 2 is
about 10 us of kernel work in 8 launches) are launch bound; replaying a graph removes that."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _step(fn, q, k, v, do):
    for t in (q, k, v):
        t.grad = None
    out = fn(q, k, v)
    out.backward(do)
    return out.detach(), q.grad, k.grad, v.grad


@pytest.mark.filterwarnings("ignore:The AccumulateGrad node's stream does not match")
@pytest.mark.parametrize("fused", [False, True])
def test_attention_step_replays_from_a_cuda_graph(fused):
    from sparse import SparseLayout, attention, matmul, softmax
    from sparse.kernel import sparse_ops
    from sparse.patterns import local_global_causal
    block, dtype = (64, torch.float16) if fused else (32, torch.float16)
    pattern = local_global_causal(1024 // block, 4, 1)
    layout = SparseLayout(pattern, block=block)
    gen = torch.Generator(device="cuda").manual_seed(9)
    q, k, v = (torch.randn(12, 1024, 64, device="cuda", generator=gen).to(dtype).requires_grad_(True) for _ in range(3))
    do = torch.randn(12, 1024, 64, device="cuda", generator=gen).to(dtype)
    if fused:
        fn = lambda a, b, c: attention(a, b, c, layout, 0.125, True)
    else:
        fn = lambda a, b, c: matmul(softmax(matmul(a, b, "sdd", layout, False, True), layout, 0.125, True), c, "dsd", layout)
    eager = [t.clone() for t in _step(fn, q, k, v, do)]
    # warm up on a side stream (allocator pools, lazy initialisation), then capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            _step(fn, q, k, v, do)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    for t in (q, k, v):
        t.grad = None
    with torch.cuda.graph(graph):
        out = fn(q, k, v)
        out.backward(do)
    captured = (out, q.grad, k.grad, v.grad)
    # new inputs in the same buffers: the replay must follow them
    with torch.no_grad():
        for t in (q, k, v):
            t.mul_(-0.5)
    reference = [t.clone() for t in _step(fn, q, k, v, do)]
    for t in captured:
        t.detach().zero_()
    graph.replay()
    torch.cuda.synchronize()
    sparse_ops.check_device_status(0)
    for name, got, ref, old in zip(("out", "dq", "dk", "dv"), captured, reference, eager):
        assert torch.equal(got, ref), name
        assert not torch.equal(got, old), name
