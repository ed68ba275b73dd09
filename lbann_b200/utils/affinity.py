"""Binding a rank to the CPU cores next to its GPU.

Pinned host buffers are placed by first touch, and the copy / collation threads run where
the process runs: a rank whose cores sit on the other socket reads its mini-batches across
the socket interconnect on every host-to-device copy.  The reference binds ranks with hwloc
(``lbann::hwloc`` in src/utils/hwloc_utils.cpp and the launcher's ``--bind-to``); here the
NUMA node of the GPU is read from sysfs (``/sys/bus/pci/devices/<id>/numa_node`` and
``local_cpulist``) and the process is restricted to those cores with ``sched_setaffinity``.
Nothing is changed when the information is missing, when the cores are not in the
process's allowed set, or when ``LBANN_DISABLE_NUMA_BIND`` is set.
"""
from __future__ import annotations

import os
from typing import Optional, Set


def parse_cpulist(text: str) -> Set[int]:
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11}."""
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


def gpu_pci_address(index: int) -> Optional[str]:
    import torch
    try:
        p = torch.cuda.get_device_properties(index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def local_cpus_of(pci_address: str, sysfs: str = "/sys/bus/pci/devices") -> Set[int]:
    try:
        with open(os.path.join(sysfs, pci_address, "local_cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return set()


def bind_to_gpu(index: int, sysfs: str = "/sys/bus/pci/devices") -> Optional[Set[int]]:
    """Restricts this process to the cores local to GPU ``index``; returns the set that was
    applied, or None when nothing was changed."""
    if os.environ.get("LBANN_DISABLE_NUMA_BIND", "") not in ("", "0"):
        return None
    if not hasattr(os, "sched_setaffinity"):
        return None
    addr = gpu_pci_address(index)
    if addr is None:
        return None
    local = local_cpus_of(addr, sysfs)
    try:
        allowed = os.sched_getaffinity(0)
    except OSError:
        return None
    target = local & allowed
    # leave it alone when the node is unknown, or when binding would leave too few cores for
    # the I/O threads of this rank
    if len(target) < 4 or target == allowed:
        return None
    try:
        os.sched_setaffinity(0, target)
    except OSError:
        return None
    return target
