"""Placement of pinned host buffers for the host-buffer calls (`hb_matmul_host`, `hb_attention_host`).

A pinned buffer whose pages sit on the other socket makes every host<->device copy cross the
socket interconnect; with one process per GPU and every process started on the same cores, all
eight ranks' buffers land on one memory controller.  `near_gpu(bus_id)` is a context manager
that asks the kernel to prefer the NUMA node the GPU's PCIe root belongs to for the pages
allocated inside it (`set_mempolicy(MPOL_PREFERRED)`), and puts the default policy back on exit.
Everything here is advisory: where sysfs has no answer, the node is not in the process's allowed
set or the system call is refused, the block runs unchanged and `.outcome` says why.
"""
from __future__ import annotations

import ctypes
import os
import platform

_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}
_MPOL_DEFAULT, _MPOL_PREFERRED = 0, 1


def parse_cpulist(text: str) -> list[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11] (the format of sysfs cpulist / nodelist files)."""
    out: list[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.extend(range(int(lo), int(hi or lo) + 1))
    return out


def normalise_bus_id(bus_id: str) -> str:
    """'00000000:1B:00.0' or '1b:00.0' -> '0000:1b:00.0', the name sysfs uses."""
    s = bus_id.strip().lower()
    parts = s.split(":")
    if len(parts) == 2:
        parts = ["0000"] + parts
    if len(parts) != 3:
        raise ValueError(f"not a PCI bus id: {bus_id!r}")
    return f"{int(parts[0], 16):04x}:{parts[1]}:{parts[2]}"


def gpu_numa_node(bus_id: str, sysfs: str = "/sys") -> int | None:
    """NUMA node of a PCI device, or None where sysfs does not say (file absent, or -1)."""
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", normalise_bus_id(bus_id), "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def online_nodes(sysfs: str = "/sys") -> list[int]:
    try:
        with open(os.path.join(sysfs, "devices/system/node/online")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


def _set_mempolicy(mode: int, node: int | None) -> int:
    nr = _SYS_SET_MEMPOLICY.get(platform.machine())
    if nr is None:
        return -1
    libc = ctypes.CDLL(None, use_errno=True)
    if node is None:
        return libc.syscall(ctypes.c_long(nr), ctypes.c_long(mode), ctypes.c_void_p(0), ctypes.c_ulong(0))
    words = node // 64 + 1
    mask = (ctypes.c_ulong * words)()
    mask[node // 64] = 1 << (node % 64)
    return libc.syscall(ctypes.c_long(nr), ctypes.c_long(mode), mask, ctypes.c_ulong(words * 64 + 1))


class near_gpu:
    """with near_gpu(bus_id) as place: ...allocate and pin...; place.outcome tells what happened."""

    def __init__(self, bus_id: str | None, sysfs: str = "/sys"):
        self.bus_id, self.sysfs = bus_id, sysfs
        self.node: int | None = None
        self.outcome = "unchanged: no bus id"
        self._set = False

    def __enter__(self):
        if self.bus_id is None:
            return self
        self.node = gpu_numa_node(self.bus_id, self.sysfs)
        nodes = online_nodes(self.sysfs)
        if self.node is None:
            self.outcome = "unchanged: sysfs names no node for the GPU"
        elif len(nodes) < 2:
            self.outcome = "unchanged: one memory node"
        elif _set_mempolicy(_MPOL_PREFERRED, self.node) != 0:
            self.outcome = f"unchanged: set_mempolicy refused (errno {ctypes.get_errno()})"
        else:
            self._set = True
            self.outcome = "preferred"
        return self

    def __exit__(self, *exc):
        if self._set:
            _set_mempolicy(_MPOL_DEFAULT, None)
            self._set = False
        return False
