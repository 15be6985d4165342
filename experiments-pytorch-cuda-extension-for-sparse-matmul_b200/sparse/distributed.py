"""Head sharding for multi-GPU runs.

Every (batch, head) slice of the block-sparse ops is independent (the reference
already treats the flattened leading dims as a grid axis,
sparse/native/sparse_smm_gpu.cu:39-41), so N GPUs each take a contiguous range
of the flattened batch*head axis and no collective is needed on the data path.
``torch.distributed`` is used only to gather per-slice checksums for
verification and to combine timings.
"""
from typing import List, Tuple

import torch


def shard_bounds(total: int, rank: int, world_size: int) -> Tuple[int, int]:
    """[begin, end) of the contiguous slice of ``total`` items owned by ``rank``; sizes differ by at most 1."""
    if not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of size %d" % (rank, world_size))
    base, extra = divmod(total, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def slice_checksums(x: torch.Tensor) -> torch.Tensor:
    """One float64 checksum per leading-dim slice: sum and sum of squares, order independent enough
    to compare runs that shard the slices differently (each slice is reduced on its own)."""
    flat = x.detach().reshape(x.shape[0], -1).double()
    return torch.stack((flat.sum(dim=1), (flat * flat).sum(dim=1)), dim=1)


def gather_slices(local: torch.Tensor, total: int) -> torch.Tensor:
    """all_gather per-slice rows (first dim = local slices) from every rank into ``[total, ...]`` order.
    Works on the default process group (gloo on CPU, nccl on GPUs); without one, returns ``local``."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = [shard_bounds(total, r, world) for r in range(world)]
    width = max(e - b for b, e in sizes)
    padded = local.new_zeros((width,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    parts: List[torch.Tensor] = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([parts[r][: e - b] for r, (b, e) in enumerate(sizes)], dim=0)
