"""Keep a rank's host threads, and with them its pinned staging memory, on the NUMA node of its GPU.

With one process per GPU on a two-socket host, pinned buffers that were first touched on the wrong socket make every
host-to-device copy cross the inter-socket link, and eight ranks copying at once share that link.  Linux places pages
on the node of the thread that first touches them, so restricting the process to the CPUs next to its GPU before it
allocates pinned memory is enough.  Everything here reads sysfs and changes only this process's CPU affinity.
"""
from __future__ import annotations

import os
from typing import Optional, Set


def _parse_cpu_list(text: str) -> Set[int]:
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a CUDA device from its PCI address, or None when the host does not say (single node, container)."""
    import torch

    props = torch.cuda.get_device_properties(device_index)
    bdf = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", bdf, "numa_node")) as fh:
            node = int(fh.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def bind_to_numa_node(node: Optional[int], sysfs: str = "/sys") -> Optional[Set[int]]:
    """Restrict this process to the CPUs of ``node`` (intersected with the CPUs it may already use).  Returns the new
    CPU set, or None when nothing was changed (unknown node, no such node, empty intersection, no affinity support)."""
    if node is None or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        with open(os.path.join(sysfs, f"devices/system/node/node{node}/cpulist")) as fh:
            cpus = _parse_cpu_list(fh.read())
    except (OSError, ValueError):
        return None
    allowed = os.sched_getaffinity(0) & cpus
    if not allowed:
        return None
    os.sched_setaffinity(0, allowed)
    return allowed


def gpu_cpu_affinity(device_index: int) -> Optional[Set[int]]:
    """The CPUs the driver names as closest to the device (NVML, read-only query), or None without NVML.  Containers
    often hide the NUMA node of a PCI device in sysfs while NVML still knows the device's CPU affinity."""
    try:
        import pynvml
        import torch

        pynvml.nvmlInit()
        try:
            props = torch.cuda.get_device_properties(device_index)
            bdf = f"{getattr(props, 'pci_domain_id', 0):08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bdf.encode())
            words = (max(os.sched_getaffinity(0) | {os.cpu_count() or 1}) + 64) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        finally:
            pynvml.nvmlShutdown()
    except Exception:      # no NVML, no such query in this driver, or a device NVML cannot see: nothing to go by
        return None
    return {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1} or None


def bind_to_gpu(device_index: int) -> Optional[int]:
    """Move this process next to its GPU.  Returns the NUMA node it now runs on, -1 when only the driver's CPU list was
    available (and used), or None when the host gave no answer or the CPUs are outside this process's allowance."""
    node = gpu_numa_node(device_index)
    if bind_to_numa_node(node):
        return node
    cpus = gpu_cpu_affinity(device_index)
    if cpus and hasattr(os, "sched_setaffinity"):
        allowed = os.sched_getaffinity(0) & cpus
        if allowed and allowed != os.sched_getaffinity(0):
            os.sched_setaffinity(0, allowed)
            return -1
    return None


__all__ = ["bind_to_gpu", "bind_to_numa_node", "gpu_cpu_affinity", "gpu_numa_node"]
