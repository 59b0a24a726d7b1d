"""Communication cost model of one NVSwitch box (and, coarsely, of Ethernet between boxes).

Per GPU, ``N`` bytes, ``P`` ranks, per-direction link bandwidth ``B``:

* NVLS all-reduce (in-switch reduction)  ``N (1 + 1/P) / B``  - each GPU's memory is read once by the switch and
  receives the full result once;
* two-shot all-reduce over peer loads/stores  ``2 N (P-1) / (P B)``;
* reduce-scatter or all-gather alone  ``N (P-1) / (P B)``;
* every collective launch pays a latency floor ``alpha`` (kernel launch + cross-GPU flag round trip).

``LinkModel.fit`` re-fits ``alpha`` and ``B`` by least squares from measured ``(bytes, seconds)`` points, e.g. the
output of ``autodist_b200.parallel.bench_comm``. Defaults are figures measured on an 8 x B200 NVSwitch box: 770 GB/s per
direction for peer copies and a 725 GB/s all-reduce bus bandwidth at 1 GiB.
"""
from dataclasses import dataclass

import numpy as np


@dataclass
class LinkModel:
    bandwidth_gbs: float = 770.0     # per direction per GPU
    alpha_us: float = 12.0           # latency floor of one fused collective launch

    def time_s(self, bytes_on_link):
        return self.alpha_us * 1e-6 + bytes_on_link / (self.bandwidth_gbs * 1e9)

    @classmethod
    def fit(cls, bytes_on_link, seconds):
        """Least-squares ``t = alpha + bytes / B`` over measured points."""
        x = np.asarray(bytes_on_link, dtype=np.float64)
        y = np.asarray(seconds, dtype=np.float64)
        A = np.stack([np.ones_like(x), x], 1)
        (alpha, inv_b), *_ = np.linalg.lstsq(A, y, rcond=None)
        alpha = max(alpha, 0.0)
        inv_b = max(inv_b, 1e-15)
        return cls(bandwidth_gbs=1.0 / inv_b / 1e9, alpha_us=alpha * 1e6)


class NVSwitchCostModel:
    def __init__(self, num_gpus, link: LinkModel = None, nvls=True, ethernet_gbps=None, num_nodes=1, hbm_gbs=6518.6):
        self.P = max(1, int(num_gpus))
        self.link = link or LinkModel()
        self.nvls = nvls
        self.num_nodes = num_nodes
        self.ethernet_gbps = ethernet_gbps
        self.hbm_gbs = hbm_gbs

    def _inter_node(self, nbytes):
        if self.num_nodes <= 1 or not self.ethernet_gbps:
            return 0.0
        # ring over nodes on the slowest NIC
        return 2.0 * nbytes * (self.num_nodes - 1) / self.num_nodes / (self.ethernet_gbps / 8.0 * 1e9)

    def all_reduce(self, nbytes):
        if self.P <= 1:
            return 0.0
        P = self.P
        on_link = nbytes * (1.0 + 1.0 / P) if self.nvls else 2.0 * nbytes * (P - 1) / P
        return self.link.time_s(on_link) + self._inter_node(nbytes)

    def reduce_scatter(self, nbytes):
        if self.P <= 1:
            return 0.0
        return self.link.time_s(nbytes * (self.P - 1) / self.P) + self._inter_node(nbytes) / 2

    all_gather = reduce_scatter

    def reduce_to_owner(self, nbytes):
        """Every rank's copy travels to one owner: the owner's ingress link is the bottleneck."""
        if self.P <= 1:
            return 0.0
        return self.link.time_s(nbytes * (self.P - 1))

    broadcast_from_owner = reduce_to_owner

    def sparse_rows(self, rows, row_bytes):
        """Row-sparse exchange: each rank sends its rows to the owners, owners spread evenly."""
        if self.P <= 1:
            return 0.0
        return self.link.time_s(rows * row_bytes * (self.P - 1) / self.P)

    def optimizer(self, numel, bytes_per_param=30.0, sharded=False):
        """Bandwidth-bound update: fp32 p, g, m, v read + p, m, v written + bf16 copy."""
        n = numel / self.P if sharded else numel
        return n * bytes_per_param / (self.hbm_gbs * 1e9)
