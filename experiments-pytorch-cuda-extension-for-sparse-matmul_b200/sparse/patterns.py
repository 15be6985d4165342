"""Generators of 2-D block patterns (int64 0/1 tensors on the CPU).

The reference takes an arbitrary pattern and ships no generator; these are
the usual block-sparse attention shapes, including the five layouts the
benchmark configurations of this library are defined on.  All random draws
use an explicit ``torch.Generator`` so a seed fixes the pattern.
"""
import torch


def _grid(rows: int, cols: int):
    i = torch.arange(rows).unsqueeze(1)
    j = torch.arange(cols).unsqueeze(0)
    return i, j


def random_with_diagonal(rows: int, cols: int, density: float, seed: int) -> torch.Tensor:
    """Bernoulli(density) blocks with the main diagonal forced on."""
    gen = torch.Generator().manual_seed(seed)
    i, j = _grid(rows, cols)
    return ((torch.rand(rows, cols, generator=gen) < density) | (i == j)).long()


def local_global_causal(size: int, window: int = 4, num_global: int = 1) -> torch.Tensor:
    """Causal local window of ``window`` blocks plus ``num_global`` global block rows / columns."""
    i, j = _grid(size, size)
    return ((j <= i) & ((i - j < window) | (j < num_global) | (i < num_global))).long()


def strided_local(size: int, stride: int = 8, window: int = 2) -> torch.Tensor:
    """Non-causal strided pattern: every ``stride``-th diagonal plus a band of half-width ``window``."""
    i, j = _grid(size, size)
    return ((((i - j) % stride) == 0) | ((i - j).abs() <= window)).long()


def bigbird(size: int, window_half: int = 1, num_global: int = 2, num_random: int = 3, seed: int = 0) -> torch.Tensor:
    """Band of half-width ``window_half``, ``num_global`` global rows / columns and, for every row
    in ascending order, ``num_random`` distinct random blocks drawn from that row's empty columns."""
    gen = torch.Generator().manual_seed(seed)
    i, j = _grid(size, size)
    pattern = (((i - j).abs() <= window_half) | (i < num_global) | (j < num_global)).long()
    for r in range(size):
        empty = torch.nonzero(pattern[r] == 0, as_tuple=False).flatten()
        if empty.numel() == 0:
            continue
        pick = empty[torch.randperm(empty.numel(), generator=gen)[:num_random]]
        pattern[r, pick] = 1
    return pattern


def causal(size: int) -> torch.Tensor:
    """Dense lower-triangular block pattern."""
    i, j = _grid(size, size)
    return (j <= i).long()


def full(rows: int, cols: int) -> torch.Tensor:
    return torch.ones(rows, cols, dtype=torch.long)
