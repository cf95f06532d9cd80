"""Pinned host staging buffers placed near the GPU that will read them.

A step that starts from host memory (a rollout worker's logits, a data loader's batch) is bound by the
host-to-device copy, and on a two-socket host that copy is slower when the pinned pages sit on the other
socket's memory: the DMA then crosses the inter-socket link and, with eight GPUs copying at once, all of
them pull from one socket's memory controllers.  Linux places pages on the node of the CPU that allocates
them, so the helpers here move the calling thread onto the CPUs of the GPU's NUMA node for the duration
of the allocation and put its affinity back afterwards.  Everything is read from sysfs; where the node is
unknown (single-node hosts, containers that hide it) the helpers do nothing.  No setting of the GPU or of
the host outlives the call; only the calling thread's own CPU mask changes, and it is restored.
"""
from __future__ import annotations

import contextlib
import os
from typing import Iterator, Optional, Set

import torch

_SYSFS = "/sys"


def parse_cpulist(text: str) -> Set[int]:
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11} (the format of sysfs `cpulist` files)."""
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def pci_address(device_index: int) -> str:
    """'dddd:bb:dd.0' of a CUDA device, as sysfs names it."""
    p = torch.cuda.get_device_properties(device_index)
    return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"


def numa_node_of(pci: str, sysfs: str = _SYSFS) -> Optional[int]:
    """NUMA node of a PCI device, or None when sysfs does not say (file missing, or -1)."""
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", pci, "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def cpus_of_node(node: int, sysfs: str = _SYSFS) -> Set[int]:
    try:
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


@contextlib.contextmanager
def near_gpu(device_index: int, sysfs: str = _SYSFS) -> Iterator[Optional[int]]:
    """Run the body on the CPUs of the GPU's NUMA node (those of them this thread may use); yields the node
    or None when nothing was changed.  The thread's CPU mask is restored on exit."""
    node, old, moved = None, None, False
    try:
        node = numa_node_of(pci_address(device_index), sysfs)
        if node is not None:
            old = os.sched_getaffinity(0)
            want = cpus_of_node(node, sysfs) & old
            if want and want != old:
                os.sched_setaffinity(0, want)
                moved = True
    except Exception:  # best effort: no CUDA device, no sysfs, a mask the kernel refuses
        moved = False
    try:
        yield node if moved else None
    finally:
        if moved:
            try:
                os.sched_setaffinity(0, old)
            except OSError:
                pass


def pinned_empty(shape, dtype, device_index: int) -> torch.Tensor:
    """Page-locked host tensor allocated while the thread sits on the GPU's NUMA node."""
    with near_gpu(device_index):
        return torch.empty(shape, dtype=dtype, pin_memory=True)
