"""Topology probe (reference: ``src/ths_op/topo_utils.cc``, ``include/flux/ths_op/topo_utils.h``):
is every pair of GPUs of the node connected by NVLink, is there an NVSwitch, how many GPUs share
a NUMA node. The reference uses the answers to choose between all-to-all, 1-D ring and 2-D ring
transfers; here they only validate that the node is the NVSwitch machine the kernels assume.
NVML is read through ``pynvml`` (read-only queries); ``nvml`` can be replaced by any object with
the same functions, which is how the CPU tests run."""
from __future__ import annotations

import glob
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

_NVLINK_MAX_LINKS = 18
_REMOTE_SWITCH = 2      # NVML_NVLINK_DEVICE_TYPE_SWITCH


@dataclass
class Topology:
    num_gpus: int = 0
    nvlink_links: List[int] = field(default_factory=list)     # active NVLink links per GPU
    has_nvlink: bool = False
    has_nvswitch: bool = False
    has_heterogeneous_nvlink: bool = False
    numa_node: List[int] = field(default_factory=list)
    pcie_gen: List[int] = field(default_factory=list)
    names: List[str] = field(default_factory=list)

    @property
    def numa_local_world_size(self) -> int:
        if not self.numa_node:
            return self.num_gpus
        counts: Dict[int, int] = {}
        for n in self.numa_node:
            counts[n] = counts.get(n, 0) + 1
        return min(counts.values())


def _numa_of(pci_bus_id: str) -> int:
    path = f"/sys/bus/pci/devices/{pci_bus_id.lower()}/numa_node"
    for cand in (path, path.replace("00000000:", "0000:")):
        try:
            with open(cand) as f:
                return max(int(f.read().strip()), 0)
        except OSError:
            continue
    return 0


def probe(nvml=None) -> Topology:
    if nvml is None:
        import pynvml as nvml  # type: ignore
    nvml.nvmlInit()
    t = Topology()
    try:
        t.num_gpus = nvml.nvmlDeviceGetCount()
        for i in range(t.num_gpus):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            name = nvml.nvmlDeviceGetName(h)
            t.names.append(name.decode() if isinstance(name, bytes) else str(name))
            active, switch = 0, False
            for link in range(_NVLINK_MAX_LINKS):
                try:
                    if not nvml.nvmlDeviceGetNvLinkState(h, link):
                        continue
                except Exception:
                    break
                active += 1
                try:
                    if nvml.nvmlDeviceGetNvLinkRemoteDeviceType(h, link) == _REMOTE_SWITCH:
                        switch = True
                except Exception:
                    pass
            t.nvlink_links.append(active)
            t.has_nvswitch = t.has_nvswitch or switch
            try:
                t.pcie_gen.append(int(nvml.nvmlDeviceGetCurrPcieLinkGeneration(h)))
            except Exception:
                t.pcie_gen.append(0)
            try:
                bus = nvml.nvmlDeviceGetPciInfo(h).busId
                t.numa_node.append(_numa_of(bus.decode() if isinstance(bus, bytes) else str(bus)))
            except Exception:
                t.numa_node.append(0)
        t.has_nvlink = t.num_gpus > 0 and all(n > 0 for n in t.nvlink_links)
        t.has_heterogeneous_nvlink = len(set(t.nvlink_links)) > 1
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass
    return t


_CACHED: Optional[Topology] = None


def topology() -> Topology:
    global _CACHED
    if _CACHED is None:
        _CACHED = probe()
    return _CACHED


def has_nvswitch() -> bool:
    return topology().has_nvswitch


def has_heterogeneous_nvlink() -> bool:
    return topology().has_heterogeneous_nvlink


def topo_numa_local_world_size() -> int:
    return topology().numa_local_world_size
