"""GPU topology of the box, read from NVML: which GPUs exist, how each pair is
connected (NVLink through NVSwitch, direct NVLink, PCIe), and which GPUs share
an NVLink fabric domain.

    python -m torchcomms_b200.utils.topology          # prints the summary
    topo = discover()                                  # Topology
    topo.nvlink_all_to_all                             # every pair reachable over NVLink
    topo.domains()                                     # [[0, 1, ..., 7]]: GPUs per fabric clique
    topo.ring_order()                                  # a rank order that keeps neighbours NVLink-connected

Only read-only NVML queries are made; nothing on the GPUs is changed.  The NVML
binding is passed in (``discover(nvml=module)``), so the logic is tested on a
machine without a GPU against a fake.

Parity: comms/prims/topology (``TopologyDiscovery`` over NVML fabric info: the
reference uses it to decide which peers are NVLink peers and which NVLink
domain a rank belongs to).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

# Pair classes, best first.
NVSWITCH = "NVSWITCH"    # NVLink through a switch: full bandwidth to every peer
NVLINK = "NVLINK"        # direct NVLink between the two GPUs
PCIE = "PCIE"            # peer access over PCIe only
NONE = "NONE"            # no peer access
SELF = "SELF"


@dataclass
class GpuInfo:
    index: int
    name: str = ""
    uuid: str = ""
    pci_bus_id: str = ""
    memory_bytes: int = 0
    nvlink_links: int = 0            # links in the active state
    nvlink_version: int = 0
    nvlink_to_switch: bool = False   # at least one active link ends at an NVSwitch
    fabric_cluster: str = ""         # NVLink fabric cluster UUID ("" when not in a fabric)
    fabric_clique: int = -1
    numa_node: int = -1


@dataclass
class Topology:
    gpus: List[GpuInfo] = field(default_factory=list)
    pairs: List[List[str]] = field(default_factory=list)     # pairs[i][j]: class of the i -> j connection
    driver_version: str = ""

    @property
    def count(self) -> int:
        return len(self.gpus)

    @property
    def nvlink_all_to_all(self) -> bool:
        """True when every pair of distinct GPUs is NVLink-connected (what the peer-memory kernels assume)."""
        n = self.count
        return n > 0 and all(self.pairs[i][j] in (NVSWITCH, NVLINK) for i in range(n) for j in range(n) if i != j)

    @property
    def has_nvswitch(self) -> bool:
        return any(g.nvlink_to_switch for g in self.gpus)

    def domains(self) -> List[List[int]]:
        """GPUs grouped by NVLink reachability (connected components of the NVLink pair graph);
        GPUs that report a fabric clique are grouped by (cluster, clique) first."""
        n = self.count
        parent = list(range(n))

        def find(x: int) -> int:
            while parent[x] != x:
                parent[x] = parent[parent[x]]
                x = parent[x]
            return x

        def union(a: int, b: int) -> None:
            ra, rb = find(a), find(b)
            if ra != rb:
                parent[max(ra, rb)] = min(ra, rb)

        by_clique: Dict[Any, int] = {}
        for g in self.gpus:
            if g.fabric_cluster and g.fabric_clique >= 0:
                key = (g.fabric_cluster, g.fabric_clique)
                if key in by_clique:
                    union(by_clique[key], g.index)
                else:
                    by_clique[key] = g.index
        for i in range(n):
            for j in range(i + 1, n):
                if self.pairs[i][j] in (NVSWITCH, NVLINK):
                    union(i, j)
        groups: Dict[int, List[int]] = {}
        for i in range(n):
            groups.setdefault(find(i), []).append(i)
        return [groups[k] for k in sorted(groups)]

    def ring_order(self) -> List[int]:
        """An order of all GPUs in which consecutive GPUs (cyclically) are NVLink-connected where the
        topology allows it.  Behind an NVSwitch any order works and the index order is returned;
        on direct-NVLink boxes a greedy walk follows the links."""
        n = self.count
        if n <= 2 or self.has_nvswitch:
            return list(range(n))
        order, left = [0], set(range(1, n))
        while left:
            cur = order[-1]
            nxt = next((j for j in sorted(left) if self.pairs[cur][j] in (NVSWITCH, NVLINK)), None)
            if nxt is None:
                nxt = min(left)
            order.append(nxt)
            left.discard(nxt)
        return order

    def summary(self) -> str:
        lines = [f"{self.count} GPU(s), driver {self.driver_version or '?'}; NVSwitch: {'yes' if self.has_nvswitch else 'no'}; "
                 f"NVLink all-to-all: {'yes' if self.nvlink_all_to_all else 'no'}; domains: {self.domains()}"]
        for g in self.gpus:
            fabric = f" fabric {g.fabric_cluster[:8]}/{g.fabric_clique}" if g.fabric_cluster else ""
            lines.append(f"  GPU{g.index} {g.name} {g.memory_bytes / 2**30:.0f} GiB  {g.pci_bus_id}  NVLink v{g.nvlink_version} x{g.nvlink_links}"
                         f"{' (switch)' if g.nvlink_to_switch else ''}{fabric}  numa {g.numa_node}")
        short = {NVSWITCH: "NVS", NVLINK: "NVL", PCIE: "PIX", NONE: " - ", SELF: " X "}
        lines.append("      " + " ".join(f"{j:>4}" for j in range(self.count)))
        for i in range(self.count):
            lines.append(f"  {i:>3} " + " ".join(f"{short[self.pairs[i][j]]:>4}" for j in range(self.count)))
        return "\n".join(lines)

    def as_dict(self) -> Dict[str, Any]:
        return {"driver_version": self.driver_version, "gpus": [g.__dict__.copy() for g in self.gpus], "pairs": self.pairs,
                "nvlink_all_to_all": self.nvlink_all_to_all, "has_nvswitch": self.has_nvswitch, "domains": self.domains()}


def _text(v: Any) -> str:
    return v.decode() if isinstance(v, bytes) else str(v)


def _try(fn, *args, default=None):
    try:
        return fn(*args)
    except Exception:  # noqa: BLE001 - NVML raises its own error types; a missing query is not fatal
        return default


_MAX_LINKS = 18   # NVLink 5: 18 links per GPU


def discover(nvml: Optional[Any] = None) -> Topology:
    """Reads the topology through ``nvml`` (default: the ``pynvml`` module)."""
    own = nvml is None
    if own:
        import pynvml as nvml  # provided by nvidia-ml-py
    nvml.nvmlInit()
    try:
        topo = Topology(driver_version=_text(_try(nvml.nvmlSystemGetDriverVersion, default="")))
        handles = []
        for i in range(nvml.nvmlDeviceGetCount()):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            handles.append(h)
            g = GpuInfo(index=i)
            g.name = _text(_try(nvml.nvmlDeviceGetName, h, default=""))
            g.uuid = _text(_try(nvml.nvmlDeviceGetUUID, h, default=""))
            pci = _try(nvml.nvmlDeviceGetPciInfo, h)
            g.pci_bus_id = _text(getattr(pci, "busId", "")) if pci is not None else ""
            mem = _try(nvml.nvmlDeviceGetMemoryInfo, h)
            g.memory_bytes = int(getattr(mem, "total", 0)) if mem is not None else 0
            g.numa_node = int(_try(getattr(nvml, "nvmlDeviceGetNumaNodeId", lambda _h: -1), h, default=-1))
            enabled = getattr(nvml, "NVML_FEATURE_ENABLED", 1)
            switch_type = getattr(nvml, "NVML_NVLINK_DEVICE_TYPE_SWITCH", 2)
            for link in range(_MAX_LINKS):
                state = _try(nvml.nvmlDeviceGetNvLinkState, h, link)
                if state is None:
                    break
                if state != enabled:
                    continue
                g.nvlink_links += 1
                g.nvlink_version = max(g.nvlink_version, int(_try(nvml.nvmlDeviceGetNvLinkVersion, h, link, default=0) or 0))
                remote = _try(getattr(nvml, "nvmlDeviceGetNvLinkRemoteDeviceType", lambda *_a: None), h, link)
                if remote == switch_type:
                    g.nvlink_to_switch = True
            fabric = _try(getattr(nvml, "nvmlDeviceGetGpuFabricInfo", lambda _h: None), h)
            if fabric is not None and getattr(fabric, "state", 0) == getattr(nvml, "NVML_GPU_FABRIC_STATE_COMPLETED", 3):
                cluster = getattr(fabric, "clusterUuid", b"")
                cluster = bytes(cluster).hex() if not isinstance(cluster, str) else cluster
                if cluster.strip("0"):
                    g.fabric_cluster = cluster
                    g.fabric_clique = int(getattr(fabric, "cliqueId", -1))
            topo.gpus.append(g)
        n = len(handles)
        caps_nvlink = getattr(nvml, "NVML_P2P_CAPS_INDEX_NVLINK", 2)
        caps_read = getattr(nvml, "NVML_P2P_CAPS_INDEX_READ", 0)
        ok = getattr(nvml, "NVML_P2P_STATUS_OK", 0)
        topo.pairs = [[SELF if i == j else NONE for j in range(n)] for i in range(n)]
        for i in range(n):
            for j in range(n):
                if i == j:
                    continue
                if _try(nvml.nvmlDeviceGetP2PStatus, handles[i], handles[j], caps_nvlink) == ok:
                    both_switch = topo.gpus[i].nvlink_to_switch and topo.gpus[j].nvlink_to_switch
                    topo.pairs[i][j] = NVSWITCH if both_switch else NVLINK
                elif _try(nvml.nvmlDeviceGetP2PStatus, handles[i], handles[j], caps_read) == ok:
                    topo.pairs[i][j] = PCIE
        return topo
    finally:
        _try(nvml.nvmlShutdown)


if __name__ == "__main__":
    print(discover().summary())
