"""How the hot path shards across ranks (one process per GPU).

Quantize shards over rows (and over K on block boundaries) with no exchange: every block is
quantised independently, so any split on whole blocks gives the unsharded result.  The GEMM
shards over rows of A (each rank a slice of the batch, W replicated) or over rows of W (column-
parallel; cut on multiples of the partial-sum block ``group_n`` so no quantisation block straddles
ranks).  Neither needs a collective on the data path.
"""
from __future__ import annotations

from typing import Tuple


def row_range(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of ``rows`` owned by ``rank``; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    q, r = divmod(rows, world)
    begin = rank * q + min(rank, r)
    return begin, begin + q + (1 if rank < r else 0)


def column_range(n: int, rank: int, world: int, multiple: int = 32) -> Tuple[int, int]:
    """[begin, end) of the N output columns owned by ``rank``, cut on multiples of ``multiple``
    (the partial-sum quantisation block) so that every rank owns whole blocks."""
    if n % multiple:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    b, e = row_range(n // multiple, rank, world)
    return b * multiple, e * multiple


def k_range(k: int, rank: int, world: int, block: int = 128) -> Tuple[int, int]:
    """[begin, end) of K owned by ``rank`` for a K split (row-parallel linear): whole quantisation
    blocks / accumulation groups per rank.  The partial outputs of such a split must then be
    summed across ranks (an all-reduce); that sum is not the reference's sequential fp16 chain,
    so only the fp32 accumulation model keeps its meaning under a K split."""
    if k % block:
        raise ValueError(f"K={k} is not a multiple of {block}")
    b, e = row_range(k // block, rank, world)
    return b * block, e * block


def bind_host_to_device(device_index: int) -> dict:
    """Keep this process's threads and its future host allocations (pinned staging buffers above
    all) on the NUMA node that the GPU's PCIe slot hangs off, so that host<->device copies do not
    cross the socket interconnect.  One process per GPU calls it once, before it allocates pinned
    memory.  Best effort and process-local: CPU affinity is narrowed to the node's CPUs that the
    process may already use, and the memory policy becomes "prefer that node"; whatever the
    platform refuses is skipped.  Returns what was done, for the caller's log."""
    import ctypes
    import os
    import platform

    import torch

    info = {"numa_node": None, "cpus_bound": 0, "mempolicy": False}
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
    except (OSError, ValueError, AttributeError, RuntimeError):
        return info
    if node < 0:
        return info
    info["numa_node"] = node
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                if part:
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
        mine = os.sched_getaffinity(0) & cpus
        if mine:
            os.sched_setaffinity(0, mine)
            info["cpus_bound"] = len(mine)
    except (OSError, ValueError, AttributeError):
        pass
    try:
        nr = {"x86_64": 238, "aarch64": 237}.get(platform.machine())
        if nr is not None and node < 64:
            libc = ctypes.CDLL(None, use_errno=True)
            mask = ctypes.c_ulong(1 << node)
            MPOL_PREFERRED = 1
            rc = libc.syscall(ctypes.c_long(nr), ctypes.c_int(MPOL_PREFERRED), ctypes.byref(mask), ctypes.c_ulong(65))
            info["mempolicy"] = rc == 0
    except (OSError, AttributeError):
        pass
    return info
