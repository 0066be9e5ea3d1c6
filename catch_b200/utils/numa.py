"""Keep a rank's host threads (and the pinned memory they allocate) on the NUMA node of its GPU.

Pinned staging buffers are placed on the node of the thread that first touches them.  With one
process per GPU and eight GPUs on a two-socket host, buffers that all land on one socket make half
of the ranks copy across the inter-socket link and share one memory controller: the per-step
host-to-device copy then stops overlapping with compute.  The reference leaves placement to the
user (its data-loader prefetch only picks a device, torch_mlu/core/utils/data_loader.py:83-139).
"""
from __future__ import annotations

import os
import subprocess
from typing import Optional


def _physical_index(device_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if ids and all(v.isdigit() for v in ids) and device_index < len(ids):
        return int(ids[device_index])
    return device_index


def gpu_numa_node(device_index: int) -> Optional[int]:
    """NUMA node of GPU ``device_index`` (None when the host does not say)."""
    try:
        out = subprocess.run(["nvidia-smi", f"--id={_physical_index(device_index)}", "--query-gpu=pci.bus_id",
                              "--format=csv,noheader"], capture_output=True, text=True, timeout=20).stdout.strip()
        if not out:
            return None
        # nvidia-smi prints an 8-digit PCI domain, sysfs uses 4 digits
        dom, rest = out.split(":", 1)
        path = f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}/numa_node"
        node = int(open(path).read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def _parse_cpulist(text: str):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def bind_to_device_node(device_index: int) -> Optional[int]:
    """Restrict the calling process to the CPUs of the GPU's NUMA node; returns the node or None.

    Call it before pinned buffers are allocated.  Does nothing when the host has one node, hides its
    topology, or the allowed CPU set would become empty."""
    node = gpu_numa_node(device_index)
    if node is None:
        return None
    try:
        cpus = _parse_cpulist(open(f"/sys/devices/system/node/node{node}/cpulist").read())
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None
