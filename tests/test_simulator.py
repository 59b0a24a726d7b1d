"""Cost model arithmetic, re-fit from measurements, strategy ranking and dataset records."""
import os

import torch

from autodist_b200.graph_item import VariableInfo
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200.simulator import LinkModel, NVSwitchCostModel, Simulator, rank_strategies
from autodist_b200.strategy import PS, AllReduce, AutoStrategy, PartitionedPS


class Item:
    def __init__(self, variables):
        self.variables = {v.name: v for v in variables}

    @property
    def trainable_var_op_to_var(self):
        return {v.op_name: v for v in self.variables.values()}


def big_model():
    f = torch.float32
    return Item([VariableInfo("emb:0", (793471, 512), f, sparse_grad=True)] +
                [VariableInfo(f"w{i}:0", (4096, 4096), f) for i in range(8)])


def test_formulas():
    m = NVSwitchCostModel(8, LinkModel(900.0, 0.0), nvls=True)
    n = 1.34e9
    assert abs(m.all_reduce(n) - n * (1 + 1 / 8) / 900e9) < 1e-9
    m2 = NVSwitchCostModel(8, LinkModel(900.0, 0.0), nvls=False)
    assert abs(m2.all_reduce(n) - 2 * n * 7 / 8 / 900e9) < 1e-9
    assert abs(m2.reduce_scatter(n) - n * 7 / 8 / 900e9) < 1e-9
    assert NVSwitchCostModel(1).all_reduce(n) == 0.0


def test_fit_recovers_alpha_and_bandwidth():
    true = LinkModel(700.0, 15.0)
    xs = [1e6, 1.6e7, 6.4e7, 2.5e8, 1e9]
    fit = LinkModel.fit(xs, [true.time_s(x) for x in xs])
    assert abs(fit.bandwidth_gbs - 700.0) < 1.0 and abs(fit.alpha_us - 15.0) < 0.5


def test_ranking_prefers_sharded_and_sparse_aware_strategies(tmp_path):
    rs = ResourceSpec.local(num_gpus=8)
    item = big_model()
    ranked = rank_strategies({"PS_one_owner": PS(reduction_devices="gpu"), "AllReduce": AllReduce(chunk_size=4),
                              "PartitionedPS": PartitionedPS(num_shards=8, reduction_devices="gpu")}, item, rs)
    names = [n for _, n, _ in ranked]
    assert names[-1] == "PS_one_owner"        # one owner's link carries everything
    auto = AutoStrategy()
    s = auto.build(item, rs)
    assert len(auto.ranking) >= 6 and s is auto.ranking[0][2]
    # strategies that move only the touched embedding rows beat the one that funnels everything through one owner
    by = {n: t for t, n, _ in auto.ranking}
    assert by["Parallax"] < by["PS"] and by["AllReduce"] < by["PS"]
    path = Simulator.record(str(tmp_path), "r.yml", s, [0.011, 0.012, 0.010])
    recs = Simulator.load_records(str(tmp_path))
    assert os.path.exists(path) and abs(recs[0]["average"] - 0.011) < 1e-9 and len(recs[0]["runtime"]) == 3


def test_predicted_against_measured_table():
    from autodist_b200.simulator.compare import compare
    out = compare("bert-tiny", 8, 5.0, {"AllReduce": 5.2, "PartitionedPS": 5.4}, fit_overlap=True)
    rows = {r["strategy"]: r for r in out["rows"]}
    assert set(rows) >= {"AllReduce", "AllReduceEF", "Parallax", "PSLoadBalancing", "PartitionedPS"}
    assert 0.0 <= out["overlap"] <= 1.0
    assert all(r["predicted_ms"] >= 5.0 and r["sync_ms"] > 0 for r in rows.values())
    assert rows["AllReduce"]["ratio"] is not None and rows["Parallax"]["ratio"] is None
    # the compressed wire is narrower but pays pack / unpack passes over HBM
    assert rows["AllReduceEF"]["sync_ms"] != rows["AllReduce"]["sync_ms"]
