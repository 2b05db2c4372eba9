"""NUMA placement: every rank process runs on the CPUs, and prefers the memory, of the NUMA node its GPU hangs off.

The reference pins its engine process to the node of the first device and spawns the workers of other nodes as separate
processes (xllm/core/platform/numa_utils.h:34-52, core/distributed_runtime/dist_manager.cpp:92-139).  Here every GPU
already has a process of its own, so each one binds itself: pinned staging buffers, the shared-memory step channel and
the scheduler's packing loop then sit on the socket whose PCIe root the GPU uses.

Everything is read from sysfs (`root` lets tests point at a fake tree); binding uses `sched_setaffinity` and the
`set_mempolicy` system call, so no libnuma is needed.  A node that cannot be determined, or that shares no CPU with the
CPUs this process may use (a container's cpuset), leaves the process as it is.
"""
from __future__ import annotations

import ctypes
import logging
import os
from typing import List, Optional, Set

log = logging.getLogger("xllm")

MPOL_DEFAULT, MPOL_PREFERRED, MPOL_BIND = 0, 1, 2
_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}


def parse_cpulist(text: str) -> List[int]:
    """`0-3,8,10-11` -> [0, 1, 2, 3, 8, 10, 11]."""
    out: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


def num_numa_nodes(root: str = "/sys") -> int:
    """Number of NUMA nodes, or -1 when the kernel exposes none."""
    d = os.path.join(root, "devices/system/node")
    try:
        n = sum(1 for e in os.listdir(d) if e.startswith("node") and e[4:].isdigit())
    except OSError:
        return -1
    return n if n > 0 else -1


def node_cpus(node: int, root: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(root, f"devices/system/node/node{node}/cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def pci_numa_node(pci_bus_id: str, root: str = "/sys") -> int:
    """NUMA node of a PCI function given as `dddd:bb:dd.f` (case-insensitive), -1 when unknown."""
    try:
        with open(os.path.join(root, "bus/pci/devices", pci_bus_id.lower(), "numa_node")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return -1


def cuda_pci_bus_id(device_index: int) -> Optional[str]:
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def device_numa_node(device_index: int, root: str = "/sys") -> int:
    bus = cuda_pci_bus_id(device_index)
    return pci_numa_node(bus, root) if bus else -1


def _set_mempolicy(mode: int, nodes: Set[int]) -> int:
    nr = _SYS_SET_MEMPOLICY.get(os.uname().machine)
    if nr is None:
        return -1
    libc = ctypes.CDLL(None, use_errno=True)
    maxnode = 1024
    mask = (ctypes.c_ulong * (maxnode // (8 * ctypes.sizeof(ctypes.c_ulong))))()
    bits = 8 * ctypes.sizeof(ctypes.c_ulong)
    for n in nodes:
        mask[n // bits] |= 1 << (n % bits)
    rc = libc.syscall(ctypes.c_long(nr), ctypes.c_int(mode), mask if nodes else None, ctypes.c_ulong(maxnode if nodes else 0))
    return 0 if rc == 0 else -ctypes.get_errno()


def bind_to_node(node: int, root: str = "/sys", pid: int = 0, set_memory: bool = True,
                 setaffinity=os.sched_setaffinity, getaffinity=os.sched_getaffinity) -> int:
    """Run process / thread `pid` (0: the caller) on the CPUs of `node` and prefer its memory.  Returns 0 on success, a
    negative value when nothing was changed (unknown node, no usable CPU, call refused)."""
    if node < 0:
        return -1
    cpus = set(node_cpus(node, root))
    try:
        allowed = set(getaffinity(pid))
    except OSError:
        allowed = set()
    usable = cpus & allowed if allowed else cpus
    if not usable:
        return -2
    try:
        setaffinity(pid, usable)
    except OSError as e:
        log.warning("NUMA: sched_setaffinity to node %d refused: %s", node, e)
        return -3
    if set_memory and pid == 0:
        rc = _set_mempolicy(MPOL_PREFERRED, {node})
        if rc != 0:
            log.info("NUMA: set_mempolicy(preferred, node %d) not applied (%d); CPU affinity is set", node, rc)
    return 0


def bind_rank_to_device(device_index: int, root: str = "/sys") -> int:
    """Bind the calling process to the NUMA node of CUDA device `device_index`.  Returns the node, or -1."""
    if num_numa_nodes(root) <= 1:
        return -1                      # one node (or none exposed): nothing to choose
    node = device_numa_node(device_index, root)
    if node < 0:
        return -1
    if bind_to_node(node, root) != 0:
        return -1
    log.info("NUMA: rank process %d bound to node %d (cuda:%d)", os.getpid(), node, device_index)
    return node
