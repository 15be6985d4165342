"""Head sharding for multi-GPU runs.

Every (batch, head) slice of the block-sparse ops is independent (the reference
already treats the flattened leading dims as a grid axis,
sparse/native/sparse_smm_gpu.cu:39-41), so N GPUs each take a contiguous range
of the flattened batch*head axis and no collective is needed on the data path.
``torch.distributed`` is used only to gather per-slice checksums for
verification and to combine timings.
"""
import os
from typing import List, Optional, Tuple

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


def parse_cpu_list(text: str) -> List[int]:
    """CPUs of a sysfs list such as ``0-27,56-83``."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_host_to_device(pci_domain: int, pci_bus: int, pci_device: int, sysfs: str = "/sys") -> Optional[int]:
    """Pins the calling process to the CPUs of the NUMA node the GPU at this PCI address hangs off, so that the
    pinned host buffers it allocates afterwards (first touch) and the threads that fill them are local to the
    GPU's PCIe root.  One process per GPU on a two-socket host otherwise puts every rank's staging memory on
    the socket the launcher happened to start on, and all ranks' copies share that socket's memory and the
    link between the sockets.  Returns the node, or None when the host gives no locality (single node,
    ``numa_node`` = -1, no sysfs, or the node's CPUs are outside this process's allowed set); never raises."""
    try:
        address = "%04x:%02x:%02x.0" % (pci_domain, pci_bus, pci_device)
        with open(os.path.join(sysfs, "bus", "pci", "devices", address, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices", "system", "node", "node%d" % node, "cpulist")) as f:
            cpus = set(parse_cpu_list(f.read()))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError):
        return None
