"""Generate the golden fixtures of this directory by EXECUTING THE REFERENCE.

Run in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own ``sparse/layout.py`` and ``sparse/matmul.py``
(unmodified; ``Tensor.cuda`` is patched to the identity because layout.py:38
moves its results to a GPU, and ``sparse.kernel`` is replaced by a recording
stand-in because importing it would JIT-compile the CUDA sources) and writes

* ``layout_<name>.json``   -- pattern, sparse_positions, row / column layouts
                              produced by the reference ``SparseLayout``;
* ``autograd_table.json``  -- for each of the 12 (mode, trans_a, trans_b)
                              forwards, the two ``sparse_matmul`` calls the
                              reference's backward issues (sparse/matmul.py:30-50).

The fixtures are small and committed; the tests never need the reference.
"""
import json
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(REPO, "experiments-pytorch-cuda-extension-for-sparse-matmul_b200", "sparse"))
import patterns  # noqa: E402  (pattern generators only; no native code involved)


def load_reference(ref_root):
    torch.Tensor.cuda = lambda self, *a, **k: self
    pkg = types.ModuleType("refsparse")
    pkg.__path__ = [os.path.join(ref_root, "sparse")]
    sys.modules["refsparse"] = pkg
    calls = []

    class Recorder:
        def sparse_matmul(self, a, b, mode, row_layout, col_layout, tr_a, tr_b):
            calls.append({"a": a.tag, "b": b.tag, "mode": mode, "trans_a": bool(tr_a), "trans_b": bool(tr_b)})
            out = torch.zeros(1)
            out.tag = "out"
            return out

    kernel = types.ModuleType("refsparse.kernel")
    kernel.sparse_ops = Recorder()
    sys.modules["refsparse.kernel"] = kernel
    import importlib
    layout = importlib.import_module("refsparse.layout")
    matmul = importlib.import_module("refsparse.matmul")
    return layout, matmul, calls


def named_patterns():
    pats = {
        "kat_4x3": torch.tensor([[1, 0, 1], [0, 1, 0], [1, 1, 0], [0, 0, 1]]),
        "single_block_3x3": torch.tensor([[0, 0, 0], [0, 1, 0], [0, 0, 0]]),
        "full_3x5": torch.ones(3, 5, dtype=torch.long),
        "empty_row_col_5x4": torch.tensor([[1, 0, 0, 1], [0, 0, 0, 0], [1, 0, 1, 1], [0, 0, 0, 1], [1, 0, 0, 0]]),
        "one_by_one": torch.ones(1, 1, dtype=torch.long),
        "cfg1_head0": patterns.random_with_diagonal(8, 8, 0.5, 1000),
        "cfg1_head1": patterns.random_with_diagonal(8, 8, 0.5, 1001),
        "cfg2_local_global_causal_32": patterns.local_global_causal(32, 4, 1),
        "cfg3_strided_local_64": patterns.strided_local(64, 8, 2),
        "cfg4_head0": patterns.random_with_diagonal(64, 64, 0.1, 4000),
        "cfg5_bigbird_128": patterns.bigbird(128, 1, 2, 3, 5000),
        "wide_2x300": (torch.arange(600).reshape(2, 300) % 7 == 0).long(),
    }
    return pats


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of the reference project>")
    ref_root = sys.argv[1]
    layout_mod, matmul_mod, calls = load_reference(ref_root)
    for name, pattern in named_patterns().items():
        lay = layout_mod.SparseLayout(pattern.long())
        fixture = {
            "source": "reference sparse/layout.py executed on CPU",
            "pattern": pattern.tolist(),
            "sparse_positions": lay.sparse_positions.tolist(),
            "row_blocks": lay.row_layout[0].tolist(), "row_table": lay.row_layout[1].tolist(),
            "col_blocks": lay.col_layout[0].tolist(), "col_table": lay.col_layout[1].tolist(),
            "dtypes": [str(lay.row_layout[0].dtype), str(lay.row_layout[1].dtype)],
        }
        with open(os.path.join(HERE, "layout_%s.json" % name), "w") as f:
            json.dump(fixture, f, separators=(",", ":"))

    class FakeLayout:
        row_layout = ("row",)
        col_layout = ("col",)

    table = []
    for mode in ("sdd", "dsd", "dds"):
        for ta in (False, True):
            for tb in (False, True):
                a = torch.zeros(1, requires_grad=True)
                b = torch.zeros(1, requires_grad=True)
                a.tag, b.tag = "a", "b"
                ctx = types.SimpleNamespace(saved_tensors=(a, b), mode=mode, layout=FakeLayout(), trans_a=ta,
                                            trans_b=tb, needs_input_grad=(True, True, False, False, False, False))
                dc = torch.zeros(1)
                dc.contiguous = lambda: dc
                dc.tag = "dc"
                del calls[:]
                matmul_mod.SparseMatMul.backward(ctx, dc)
                table.append({"forward": {"mode": mode, "trans_a": ta, "trans_b": tb},
                              "da": dict(calls[0]), "db": dict(calls[1])})
    with open(os.path.join(HERE, "autograd_table.json"), "w") as f:
        json.dump({"source": "reference sparse/matmul.py backward executed with a recording sparse_ops",
                   "table": table}, f, indent=1)
    print("wrote", len(named_patterns()), "layout fixtures and the autograd table")


if __name__ == "__main__":
    main()
