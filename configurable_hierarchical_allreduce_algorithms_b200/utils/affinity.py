"""Host affinity for one-rank-per-GPU processes: run on the cores, and allocate on the memory node,
nearest to the rank's GPU, so that pinned staging buffers are first touched there.

Only the calling process's own CPU mask and memory policy are changed (``sched_setaffinity``,
``set_mempolicy``); nothing of the GPU or of other processes is touched.  On a machine that exposes a
single memory node (or none for the GPU) this is a no-op, and the returned record says so.

The reference leaves placement to its launcher (``mpiexec --cpu-bind depth``,
testing/custom_implementations/work_dir/all_reduce/runner_polaris_allreduce.sh:23).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path


def parse_cpulist(text: str) -> list[int]:
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def gpu_pci_address(device_index: int) -> str | None:
    try:
        import torch

        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:  # noqa: BLE001 - no CUDA, or a torch without these fields
        return None


def numa_of_pci(addr: str, sysfs_root: str = "/sys") -> tuple[int, list[int]]:
    """(memory node, cpus of that node) of a PCI device; node -1 when the platform does not say."""
    dev = Path(sysfs_root) / "bus" / "pci" / "devices" / addr
    try:
        node = int((dev / "numa_node").read_text().strip())
    except (OSError, ValueError):
        return -1, []
    if node < 0:
        return -1, []
    try:
        cpus = parse_cpulist((Path(sysfs_root) / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text())
    except OSError:
        cpus = []
    return node, cpus


def count_nodes(sysfs_root: str = "/sys") -> int:
    try:
        return len([p for p in (Path(sysfs_root) / "devices" / "system" / "node").iterdir()
                    if p.name.startswith("node") and p.name[4:].isdigit()])
    except OSError:
        return 0


def _set_mempolicy_preferred(node: int) -> bool:
    """MPOL_PREFERRED on `node` for this thread's future allocations (Linux x86-64 / aarch64 syscall)."""
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        nr = {"x86_64": 238, "aarch64": 237}.get(os.uname().machine)
        if nr is None:
            return False
        mask = ctypes.c_ulong(1 << node)
        rc = libc.syscall(nr, 1, ctypes.byref(mask), ctypes.c_ulong(8 * ctypes.sizeof(ctypes.c_ulong)))
        return rc == 0
    except Exception:  # noqa: BLE001
        return False


def bind_to_gpu(device_index: int, sysfs_root: str = "/sys", apply: bool = True, pci_addr: str | None = None) -> dict:
    """Bind the calling process to the cores and memory node of its GPU.  Returns what was found and done."""
    addr = pci_addr or gpu_pci_address(device_index)
    rec = {"pci": addr, "numa_node": -1, "nodes": count_nodes(sysfs_root), "cpus": 0, "bound": False, "mempolicy": False}
    if not addr:
        return rec
    node, cpus = numa_of_pci(addr, sysfs_root)
    rec["numa_node"], rec["cpus"] = node, len(cpus)
    if node < 0 or not cpus or rec["nodes"] < 2:
        rec["why_not"] = "the platform exposes one memory node (or none for this GPU): nothing to choose"
        return rec
    if apply:
        try:
            allowed = os.sched_getaffinity(0)
            want = allowed & set(cpus)
            if want:
                os.sched_setaffinity(0, want)
                rec["bound"] = True
                rec["cpus"] = len(want)
        except OSError:
            pass
        rec["mempolicy"] = _set_mempolicy_preferred(node)
    return rec
