"""Launch-environment helpers (reference: python/hxccl_torch/launch.py:4-12)."""
from __future__ import annotations

import os


def fill_env_from_openmpi() -> None:
    """Under mpirun, derive torch.distributed's variables from Open MPI's; set the default
    rendezvous address and port when nothing else did."""
    for ompi, ours in (("OMPI_COMM_WORLD_RANK", "RANK"), ("OMPI_COMM_WORLD_SIZE", "WORLD_SIZE"),
                       ("OMPI_COMM_WORLD_LOCAL_RANK", "LOCAL_RANK")):
        if ompi in os.environ:
            os.environ.setdefault(ours, os.environ[ompi])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_cpus(pci_bus_id: str, sysfs: str = "/sys") -> set:
    """CPUs of the NUMA node a GPU hangs off, from sysfs (`pci_bus_id` like "0000:1b:00.0").
    Empty when the machine has one node, the node is unknown (-1) or sysfs says nothing."""
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", pci_bus_id.lower(), "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return set()
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


def bind_to_gpu_numa(device_index: int) -> dict:
    """Restricts this process to the CPUs next to its GPU, so that host buffers it allocates and
    pins afterwards land in the memory that GPU reaches without crossing sockets (host-to-device
    copies of several ranks at once otherwise share one socket's memory and the inter-socket
    link). One rank per GPU calls this before it allocates pinned memory. Best effort: returns
    {"bound": False, ...} and changes nothing where the topology is flat or cannot be read."""
    info = {"bound": False, "cpus": 0, "pci": None}
    try:
        import torch  # noqa: PLC0415

        p = torch.cuda.get_device_properties(device_index)
        pci = f"{getattr(p, 'pci_domain_id', 0):04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        info["pci"] = pci
        allowed = os.sched_getaffinity(0)
        cpus = gpu_numa_cpus(pci) & allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            info.update(bound=True, cpus=len(cpus))
    except Exception as e:  # noqa: BLE001  (no sysfs, no such attribute, not permitted)
        info["why"] = repr(e)[:100]
    return info
