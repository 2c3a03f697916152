"""Topology discovery against a fake NVML (no GPU): an NVSwitch box, a box of
two direct-NVLink islands joined by PCIe, and missing queries."""
from types import SimpleNamespace

import pytest


class FakeNvml:
    NVML_FEATURE_ENABLED = 1
    NVML_NVLINK_DEVICE_TYPE_SWITCH = 2
    NVML_NVLINK_DEVICE_TYPE_GPU = 0
    NVML_P2P_CAPS_INDEX_READ = 0
    NVML_P2P_CAPS_INDEX_NVLINK = 2
    NVML_P2P_STATUS_OK = 0
    NVML_GPU_FABRIC_STATE_COMPLETED = 3

    def __init__(self, n, nvlink_pairs, switch, links=18, fabric=None, pcie_all=True, drop=()):
        self.n, self.nvlink_pairs, self.switch, self.links = n, nvlink_pairs, switch, links
        self.fabric, self.pcie_all, self.inits = fabric, pcie_all, 0
        for name in drop:                       # queries an older driver does not have
            setattr(self, name, self._unsupported)

    def _unsupported(self, *a):
        raise RuntimeError("not supported")

    def nvmlInit(self):
        self.inits += 1

    def nvmlShutdown(self):
        self.inits -= 1

    def nvmlSystemGetDriverVersion(self):
        return b"580.00"

    def nvmlDeviceGetCount(self):
        return self.n

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetName(self, h):
        return b"NVIDIA B200"

    def nvmlDeviceGetUUID(self, h):
        return f"GPU-{h:04d}"

    def nvmlDeviceGetPciInfo(self, h):
        return SimpleNamespace(busId=f"0000:{h:02x}:00.0".encode())

    def nvmlDeviceGetMemoryInfo(self, h):
        return SimpleNamespace(total=180 << 30)

    def nvmlDeviceGetNumaNodeId(self, h):
        return h // 4

    def nvmlDeviceGetNvLinkState(self, h, link):
        if link >= self.links:
            raise RuntimeError("invalid link")
        return 1 if link % 2 == 0 or self.switch else 0     # direct boxes: half of the links are down

    def nvmlDeviceGetNvLinkVersion(self, h, link):
        return 5

    def nvmlDeviceGetNvLinkRemoteDeviceType(self, h, link):
        return self.NVML_NVLINK_DEVICE_TYPE_SWITCH if self.switch else self.NVML_NVLINK_DEVICE_TYPE_GPU

    def nvmlDeviceGetGpuFabricInfo(self, h):
        if self.fabric is None:
            raise RuntimeError("not supported")
        return SimpleNamespace(state=3, clusterUuid=bytes([0xAB] * 16), cliqueId=self.fabric[h])

    def nvmlDeviceGetP2PStatus(self, a, b, index):
        if index == self.NVML_P2P_CAPS_INDEX_NVLINK:
            return 0 if (min(a, b), max(a, b)) in self.nvlink_pairs else 4
        return 0 if self.pcie_all else 4


def _all_pairs(n):
    return {(i, j) for i in range(n) for j in range(i + 1, n)}


def test_nvswitch_box():
    from torchcomms_b200.utils import topology as T

    nvml = FakeNvml(8, _all_pairs(8), switch=True, fabric=[7] * 8)
    topo = T.discover(nvml)
    assert nvml.inits == 0                                   # init / shutdown balanced
    assert topo.count == 8 and topo.driver_version == "580.00"
    assert topo.nvlink_all_to_all and topo.has_nvswitch
    assert all(topo.pairs[i][j] == (T.SELF if i == j else T.NVSWITCH) for i in range(8) for j in range(8))
    g = topo.gpus[5]
    assert (g.nvlink_links, g.nvlink_version, g.nvlink_to_switch, g.fabric_clique, g.numa_node) == (18, 5, True, 7, 1)
    assert g.name == "NVIDIA B200" and g.pci_bus_id == "0000:05:00.0" and g.memory_bytes == 180 << 30
    assert topo.domains() == [list(range(8))] and topo.ring_order() == list(range(8))
    text = topo.summary()
    assert "NVLink all-to-all: yes" in text and "NVS" in text and "GPU7" in text
    assert topo.as_dict()["domains"] == [list(range(8))]


def test_two_nvlink_islands_joined_by_pcie():
    from torchcomms_b200.utils import topology as T

    # 0-1-3-2 form a ring of direct links (no 0-3, no 1-2); 4..7 are fully connected; islands meet over PCIe
    pairs = {(0, 1), (1, 3), (2, 3), (0, 2)} | {(i, j) for i in range(4, 8) for j in range(i + 1, 8)}
    topo = T.discover(FakeNvml(8, pairs, switch=False))
    assert not topo.nvlink_all_to_all and not topo.has_nvswitch
    assert topo.pairs[0][1] == T.NVLINK and topo.pairs[0][3] == T.PCIE and topo.pairs[3][4] == T.PCIE
    assert topo.gpus[0].nvlink_links == 9 and topo.gpus[0].fabric_cluster == ""
    assert topo.domains() == [[0, 1, 2, 3], [4, 5, 6, 7]]
    order = topo.ring_order()
    assert sorted(order) == list(range(8)) and order[:4] == [0, 1, 3, 2]   # follows the links inside the island


def test_missing_queries_and_no_peer_access():
    from torchcomms_b200.utils import topology as T

    nvml = FakeNvml(2, set(), switch=False, pcie_all=False,
                    drop=("nvmlDeviceGetNumaNodeId", "nvmlDeviceGetNvLinkRemoteDeviceType", "nvmlDeviceGetPciInfo"))
    topo = T.discover(nvml)
    assert topo.pairs == [[T.SELF, T.NONE], [T.NONE, T.SELF]] and topo.domains() == [[0], [1]]
    assert topo.gpus[0].numa_node == -1 and topo.gpus[0].pci_bus_id == "" and not topo.nvlink_all_to_all
    assert T.discover(FakeNvml(0, set(), switch=False)).nvlink_all_to_all is False


def test_clock_sampler_summary_and_missing_tool(monkeypatch):
    """The sampler parses nvidia-smi rows into median clock and throttle reasons, and is inert where the tool is absent."""
    from torchcomms_b200.utils.clocks import ClockSampler

    s = ClockSampler(0)
    s.rows = [
        ["0", "1965", "1965", "412.1", "0x0000000000000000", "Not Active", "Not Active", "Not Active", "Not Active"],
        ["0", "1410", "1965", "998.7", "0x0000000000000004", "Not Active", "Not Active", "Not Active", "Active"],
        ["0", "1395", "1965", "1001.2", "0x0000000000000004", "Not Active", "Not Active", "Not Active", "Active"],
        ["0", "[N/A]", "1965", "x", "", "", "", "", ""],
    ]
    out = s.summary()
    assert out == {"sm_mhz": 1410.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    monkeypatch.setenv("PATH", "/nonexistent")
    with ClockSampler(0) as absent:
        pass
    assert absent.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
