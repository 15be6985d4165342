import json
import os
import sys

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(REPO, "experiments-pytorch-cuda-extension-for-sparse-matmul_b200")
GOLDEN = os.path.join(REPO, "tests", "golden")
for path in (PKG, REPO):
    if path not in sys.path:
        sys.path.insert(0, path)

# Tolerances of the parity contract: the largest absolute difference divided
# by the largest absolute value of the masked-dense CPU result.
TOL = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 3e-2}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_layout_names():
    return sorted(f[len("layout_"):-len(".json")] for f in os.listdir(GOLDEN)
                  if f.startswith("layout_") and f.endswith(".json"))


def load_golden_layout(name):
    with open(os.path.join(GOLDEN, "layout_%s.json" % name)) as f:
        return json.load(f)


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.numel() == 0:
        return 0.0
    assert torch.isfinite(got).all(), "non-finite values in the result"
    denom = ref.abs().max().clamp_min(1e-30)
    return float((got - ref).abs().max() / denom)


def assert_close(got, ref, dtype, what=""):
    err = rel_err(got, ref)
    assert err <= TOL[dtype], "%s: relative error %.3e exceeds %.1e" % (what, err, TOL[dtype])


def seeded(shape, seed, dtype=torch.float32, dist="normal"):
    """CPU tensor drawn in fp32 from a seeded generator, then rounded to dtype (so the
    oracle and the GPU see the same bits)."""
    gen = torch.Generator().manual_seed(seed)
    if dist == "normal":
        x = torch.randn(shape, generator=gen, dtype=torch.float32)
    else:
        x = torch.rand(shape, generator=gen, dtype=torch.float32) * 2 - 1
    return x.to(dtype)
