"""CPU tests of the host side: the C-ABI library loads and exports what include/bsa.h declares,
argument validation returns the documented codes without touching a GPU, the autograd wiring
issues exactly the calls the reference's backward issues, and head sharding is world-size
independent (2 gloo ranks)."""
import ctypes
import json
import os
import re
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

from conftest import GOLDEN, PKG, REPO, seeded
from oracle import oracle

LIB = os.path.join(PKG, "libbsa_b200.so")
HEADER = os.path.join(REPO, "include", "bsa.h")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        sys.path.insert(0, PKG)
        import build
        build.build_kernel_library()
    return ctypes.CDLL(LIB)


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert "bsa_matmul" in names and "bsa_softmax_forward" in names and "bsa_layout_build" in names
    for name in names:
        assert hasattr(lib, name), "include/bsa.h declares %s but the library does not export it" % name


def test_version_and_status_strings(lib):
    assert lib.bsa_version() >= 100
    lib.bsa_status_string.restype = ctypes.c_char_p
    assert lib.bsa_status_string(0) == b"ok"
    seen = {lib.bsa_status_string(i) for i in range(0, 12)}
    assert len(seen) == 12 and b"unknown status" not in seen
    assert lib.bsa_status_string(99) == b"unknown status"


def _matmul(lib, mode=0, dtype=1, a=16, b=16, c=16, blocks=16, table=16, nnz=1, groups=1, batches=1,
            m=64, n=64, k=64, block=64, ws=16, ws_bytes=256, engine=0):
    lib.bsa_matmul.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 6 + \
        [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    return lib.bsa_matmul(mode, dtype, 0, 0, a, b, c, blocks, table, nnz, groups, batches, m, n, k, block,
                          ws, ws_bytes, engine, None)


def test_matmul_validation_codes(lib):
    # all of these are rejected on the host before any CUDA call (the pointers are fake)
    assert _matmul(lib, mode=3) == 2                   # BSA_ERR_BAD_MODE
    assert _matmul(lib, dtype=7) == 3                  # BSA_ERR_BAD_DTYPE
    assert _matmul(lib, block=48) == 5                 # BSA_ERR_BAD_BLOCK
    assert _matmul(lib, a=None) == 1                   # BSA_ERR_NULL_POINTER
    assert _matmul(lib, ws=None) == 7                  # BSA_ERR_WORKSPACE
    assert _matmul(lib, ws_bytes=8) == 7
    assert _matmul(lib, m=96) == 4                     # BSA_ERR_BAD_SHAPE: m != groups * block
    assert _matmul(lib, k=0) == 4
    assert _matmul(lib, a=24) == 6                     # BSA_ERR_ALIGNMENT
    assert _matmul(lib, batches=70000) == 10           # BSA_ERR_TOO_LARGE
    assert _matmul(lib, batches=0) == 0                # nothing to do is not an error


def test_softmax_and_layout_validation_codes(lib):
    lib.bsa_softmax_forward.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    f = lib.bsa_softmax_forward
    assert f(1, None, 16, 16, 16, 1, 1, 1, 64, 1.0, 0, None, 0, 0, 0, None) == 1
    assert f(9, 16, 16, 16, 16, 1, 1, 1, 64, 1.0, 0, None, 0, 0, 0, None) == 3
    assert f(1, 16, 16, 16, 16, 1, 1, 1, 48, 1.0, 0, None, 0, 0, 0, None) == 5
    assert f(1, 16, 24, 16, 16, 1, 1, 1, 64, 1.0, 0, None, 0, 0, 0, None) == 6
    assert f(1, 16, 16, 16, 16, 1, 1, 3, 64, 1.0, 0, 16, 2, 64, 0, None) == 4     # 2 mask rows do not divide 3
    lib.bsa_layout_build.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int] + \
        [ctypes.c_void_p] * 6
    g = lib.bsa_layout_build
    assert g(None, 0, 2, 2, 16, 16, 16, 16, 16, None) == 1
    assert g(16, 0, 0, 2, 16, 16, 16, 16, 16, None) == 4
    assert g(16, 0, 70000, 2, 16, 16, 16, 16, 16, None) == 10
    assert g(16, 9, 2, 2, 16, 16, 16, 16, 16, None) == 3


def test_attention_validation_codes(lib):
    f = lib.bsa_attention_forward
    f.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_int64] * 5 + \
        [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]

    def call(dtype=1, q=16, o=16, lse=16, blocks=16, nnz=1, rows=1, cols=1, batches=1, d=64, block=64,
             kpm=None, kpm_batches=0, kpm_stride=0, ws=16, ws_bytes=256):
        return f(dtype, q, 16, 16, o, lse, blocks, 16, nnz, rows, cols, batches, d, block, 1.0, 0,
                 kpm, kpm_batches, kpm_stride, 0, ws, ws_bytes, None)

    # rejected on the host before any CUDA call (the pointers are fake)
    assert call(dtype=9) == 3                      # BSA_ERR_BAD_DTYPE
    assert call(dtype=0) == 3                      # fp32 has no fused kernel: callers compose the unfused ops
    assert call(block=48) == 5                     # BSA_ERR_BAD_BLOCK
    assert call(block=32) == 4                     # BSA_ERR_BAD_SHAPE: only block 64 is fused
    assert call(d=96) == 4
    assert call(q=None) == 1                       # BSA_ERR_NULL_POINTER
    assert call(ws=None) == 7                      # BSA_ERR_WORKSPACE
    assert call(q=24) == 6                         # BSA_ERR_ALIGNMENT
    assert call(nnz=5) == 4                        # more blocks than the 1 x 1 grid holds
    assert call(batches=70000) == 10               # BSA_ERR_TOO_LARGE
    assert call(kpm=16, kpm_batches=2, kpm_stride=64, batches=3) == 4
    assert call(kpm=16, kpm_batches=1, kpm_stride=32) == 4      # mask shorter than the key sequence
    assert call(batches=0) == 0                    # nothing to do is not an error
    assert call(lse=None, batches=0) == 0          # the log-sum-exp output is optional


class OracleOps:
    """CPU stand-in for the native binding (the oracle as the engine), recording every call."""

    def __init__(self, pattern, block):
        self.pattern, self.block, self.calls = pattern, block, []

    def sparse_matmul(self, a, b, mode, row_layout, col_layout, tr_a, tr_b, block):
        self.calls.append({"mode": mode, "trans_a": bool(tr_a), "trans_b": bool(tr_b)})
        return oracle.sparse_matmul(a, b, mode, self.pattern, block, tr_a, tr_b, dtype=torch.float64)


@pytest.mark.parametrize("mode", ["sdd", "dsd", "dds"])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_autograd_wiring_issues_the_reference_calls(mode, ta, tb, monkeypatch):
    import sparse
    from sparse import kernel
    from test_oracle import _operands
    pattern = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 0], [0, 0, 1]])
    block = 4
    ops = OracleOps(pattern, block)
    monkeypatch.setattr(kernel, "sparse_ops", ops)
    layout = types.SimpleNamespace(row_layout=("row",), col_layout=("col",), block=block)
    a, b = _operands(mode, ta, tb, pattern, block, 8, 13)
    a.requires_grad_(True)
    b.requires_grad_(True)
    out = sparse.matmul(a, b, mode, layout, ta, tb)
    dc = seeded(tuple(out.shape), 17).double()
    out.backward(dc)
    with open(os.path.join(GOLDEN, "autograd_table.json")) as f:
        row = next(r for r in json.load(f)["table"] if r["forward"] == {"mode": mode, "trans_a": ta, "trans_b": tb})
    assert ops.calls[0] == {"mode": mode, "trans_a": ta, "trans_b": tb}
    for got, name in zip(ops.calls[1:], ("da", "db")):
        assert got == {k: row[name][k] for k in ("mode", "trans_a", "trans_b")}, name
    # and the gradients are those of dense autograd
    ad, bd = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    a_full = oracle.to_dense(ad, pattern, block) if mode[1] == "s" else ad
    b_full = oracle.to_dense(bd, pattern, block) if mode[2] == "s" else bd
    c = (a_full.transpose(-1, -2) if ta else a_full) @ (b_full.transpose(-1, -2) if tb else b_full)
    if mode[0] == "s":
        c = oracle.to_sparse(c, pattern, block)
    c.backward(dc)
    assert torch.allclose(a.grad, ad.grad, atol=1e-10) and torch.allclose(b.grad, bd.grad, atol=1e-10)


def test_matmul_rejects_unknown_mode():
    import sparse
    layout = types.SimpleNamespace(row_layout=("row",), col_layout=("col",), block=32)
    with pytest.raises(ValueError):
        sparse.matmul(torch.zeros(1, 32, 32), torch.zeros(1, 32, 32), "ssd", layout)


def test_layout_constructor_validation():
    from sparse import SparseLayout
    with pytest.raises(ValueError):
        SparseLayout(torch.ones(2, 2, 2))
    with pytest.raises(ValueError):
        SparseLayout(torch.ones(2, 2), block=48)


def test_shard_bounds_partition():
    from sparse.distributed import shard_bounds
    for total in (0, 1, 7, 64, 512):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 4, 4)


_WORKER = r"""
import os, sys
sys.path.insert(0, {pkg!r}); sys.path.insert(0, {repo!r})
import numpy as np, torch, torch.distributed as dist
from oracle import oracle
from sparse.distributed import shard_bounds, slice_checksums, gather_slices
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size={world})
pattern = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 0]])
total = 5
b, e = shard_bounds(total, dist.get_rank(), {world})
outs = []
for head in range(b, e):                      # inputs are seeded by GLOBAL head index
    g = torch.Generator().manual_seed(100 + head)
    q = torch.randn(1, 12, 8, generator=g); k = torch.randn(1, 12, 8, generator=g)
    outs.append(oracle.sparse_matmul(q, k, "sdd", pattern, 4, False, True))
local = slice_checksums(torch.cat(outs)) if outs else torch.zeros(0, 2, dtype=torch.float64)
full = gather_slices(local, total)
if dist.get_rank() == 0:
    torch.save(full, {out!r})
dist.barrier(); dist.destroy_process_group()
"""


def test_head_sharding_is_world_size_independent(tmp_path):
    """Two gloo ranks each compute their contiguous head range; the gathered per-head checksums equal
    the single-process result."""
    from sparse.distributed import slice_checksums
    pattern = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 0]])
    outs = []
    for head in range(5):
        g = torch.Generator().manual_seed(100 + head)
        q = torch.randn(1, 12, 8, generator=g)
        k = torch.randn(1, 12, 8, generator=g)
        outs.append(oracle.sparse_matmul(q, k, "sdd", pattern, 4, False, True))
    expect = slice_checksums(torch.cat(outs))
    out = str(tmp_path / "gathered.pt")
    port = 29500 + os.getpid() % 2000
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(pkg=PKG, repo=REPO, port=port, world=2, out=out))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)]) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=180) == 0
    got = torch.load(out)
    assert torch.equal(got, expect)


def test_attention_backward_validation_codes(lib):
    f = lib.bsa_attention_backward
    f.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 13 + [ctypes.c_int64] * 5 + \
        [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]

    def call(dtype=1, q=16, dq=16, lse=16, col_blocks=16, nnz=1, rows=1, cols=1, batches=1, d=64, block=64,
             kpm=None, kpm_batches=0, kpm_stride=0, stats=16, stats_bytes=512, ws=16, ws_bytes=256):
        return f(dtype, q, 16, 16, 16, 16, lse, dq, 16, 16, 16, 16, col_blocks, 16, nnz, rows, cols, batches, d, block,
                 1.0, 0, kpm, kpm_batches, kpm_stride, 0, stats, stats_bytes, ws, ws_bytes, None)

    # rejected on the host before any CUDA call (the pointers are fake)
    assert call(dtype=9) == 3                      # BSA_ERR_BAD_DTYPE
    assert call(dtype=0) == 3                      # fp32 has no fused kernel
    assert call(block=48) == 5                     # BSA_ERR_BAD_BLOCK
    assert call(block=32) == 4                     # BSA_ERR_BAD_SHAPE: only block 64 is fused
    assert call(d=96) == 4
    assert call(q=None) == 1                       # BSA_ERR_NULL_POINTER
    assert call(lse=None) == 1
    assert call(col_blocks=None) == 1
    assert call(ws=None) == 7                      # BSA_ERR_WORKSPACE
    assert call(stats=None) == 7
    assert call(stats_bytes=511) == 7              # 1 batch x 64 rows x 8 bytes are needed
    assert call(dq=24) == 6                        # BSA_ERR_ALIGNMENT
    assert call(nnz=5) == 4
    assert call(batches=70000, stats_bytes=1 << 40) == 10     # BSA_ERR_TOO_LARGE
    assert call(kpm=16, kpm_batches=2, kpm_stride=64, batches=3, stats_bytes=4096) == 4


def test_debug_checks_flag_is_off_by_default_and_check_passes_cpu_tensors_through():
    """`sparse.kernel.check` is the opt-in status check the autograd ops call: off unless `debug_checks` (or
    BSA_DEBUG_CHECKS=1) is set, and it never touches tensors that are not on a GPU."""
    import importlib
    import os
    kernel = importlib.import_module("sparse.kernel")
    assert kernel.debug_checks == (os.environ.get("BSA_DEBUG_CHECKS", "0") not in ("", "0"))
    t = torch.zeros(3)
    old = kernel.debug_checks
    try:
        kernel.debug_checks = True
        assert kernel.check(t) is t and kernel.check(None) is None
    finally:
        kernel.debug_checks = old


def test_bind_host_to_device_reads_the_numa_node_of_the_pci_address(tmp_path, monkeypatch):
    """The host-side binding of a rank to its GPU's NUMA node, against a fake sysfs tree: the node comes from
    <sysfs>/bus/pci/devices/<address>/numa_node, its CPUs from <sysfs>/devices/system/node/node<N>/cpulist, and
    only CPUs this process may use are kept.  No locality (node -1, missing files, no usable CPU) binds nothing."""
    import importlib
    distributed = importlib.import_module("sparse.distributed")
    assert distributed.parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    allowed = sorted(os.sched_getaffinity(0))
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    (node / "cpulist").write_text("%d,100000-100003\n" % allowed[0])
    bound = {}
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: bound.update(pid=pid, cpus=set(cpus)))
    assert distributed.bind_host_to_device(0, 0x1b, 0, sysfs=str(tmp_path)) == 1
    assert bound == {"pid": 0, "cpus": {allowed[0]}}
    bound.clear()
    (node / "cpulist").write_text("100000-100003\n")                 # none of the node's CPUs is usable here
    assert distributed.bind_host_to_device(0, 0x1b, 0, sysfs=str(tmp_path)) is None and not bound
    (dev / "numa_node").write_text("-1\n")                           # the platform reports no locality
    assert distributed.bind_host_to_device(0, 0x1b, 0, sysfs=str(tmp_path)) is None and not bound
    assert distributed.bind_host_to_device(0, 0x2c, 0, sysfs=str(tmp_path)) is None and not bound   # unknown device
