"""Table-driven expectations for the eight builders on the small sparse+dense model
``emb[10000,16] (sparse), w1[16,16], b1[16], w2[16,1], b2[1]`` on ``localhost, gpus [0,1]``."""
import os

import pytest
import torch

from autodist_b200.graph_item import VariableInfo
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200.strategy import (PS, AllReduce, Parallax, PartitionedAR, PartitionedPS, PSLoadBalancing,
                                    RandomAxisPartitionAR, UnevenPartitionedPS)
from autodist_b200.strategy._placement import first_non_divisor_shards, min_divisor_shards
from autodist_b200.kernel.partitioner import split_sizes

SPECS = os.path.join(os.path.dirname(__file__), "resource_specs")


class FakeItem:
    def __init__(self, variables):
        self._vars = variables

    @property
    def trainable_var_op_to_var(self):
        return {v.op_name: v for v in self._vars}

    @property
    def variables(self):
        return {v.name: v for v in self._vars}


def model():
    f = torch.float32
    return FakeItem([
        VariableInfo("emb:0", (10000, 16), f, sparse_grad=True),
        VariableInfo("w1:0", (16, 16), f), VariableInfo("b1:0", (16,), f),
        VariableInfo("w2:0", (16, 1), f), VariableInfo("b2:0", (1,), f)])


@pytest.fixture
def r0():
    return ResourceSpec(os.path.join(SPECS, "r0.yml"))


@pytest.mark.parametrize("n,md,fnd,sizes", [
    (3, 3, 2, [2, 1]), (7, 7, 2, [4, 3]), (16, 2, 3, [6, 5, 5]), (64, 2, 3, [22, 21, 21]),
    (1000, 2, 3, [334, 333, 333]), (1024, 2, 3, [342, 341, 341]), (4096, 2, 3, [1366, 1365, 1365]),
    (10000, 2, 3, [3334, 3333, 3333]), (25088, 2, 3, [8363, 8363, 8362]),
    (30522, 2, 4, [7631, 7631, 7630, 7630]), (793471, 7, 2, [396736, 396735])])
def test_shard_count_rules(n, md, fnd, sizes):
    assert min_divisor_shards(n) == md
    assert first_non_divisor_shards(n) == fnd
    assert split_sizes(n, fnd) == sizes


def test_ps_and_pslb(r0):
    for builder in (PS(), PSLoadBalancing(local_proxy_variable=True)):
        s = builder.build(model(), r0)
        assert list(s.graph_config.replicas) == ["localhost:GPU:0", "localhost:GPU:1"]
        assert [n.var_name for n in s.node_config] == ["emb:0", "w1:0", "b1:0", "w2:0", "b2:0"]
        for n in s.node_config:
            assert n.PSSynchronizer.reduction_destination == "localhost:CPU:0"
            assert n.PSSynchronizer.sync and n.PSSynchronizer.staleness == 0
    assert s.node_config[0].PSSynchronizer.local_replication


def test_pslb_balances_bytes():
    rs = ResourceSpec(os.path.join(SPECS, "r6.yml"))   # four CPU devices
    s = PSLoadBalancing().build(model(), rs)
    dests = [n.PSSynchronizer.reduction_destination for n in s.node_config]
    assert len(set(dests)) == 4 and dests[0] != dests[1]


def test_pslb_gpu_owners(r0):
    s = PSLoadBalancing(reduction_devices="gpu").build(model(), r0)
    dests = [n.PSSynchronizer.reduction_destination for n in s.node_config]
    assert dests[0] == "localhost:GPU:0" and dests[1] == "localhost:GPU:1"


def test_staleness_needs_sync():
    with pytest.raises(AssertionError):
        PS(sync=False, staleness=2)
    with pytest.raises(AssertionError):
        PartitionedPS(sync=False, staleness=2)


def test_partitioned_ps(r0):
    s = PartitionedPS().build(model(), r0)
    by = {n.var_name: n for n in s.node_config}
    assert by["emb:0"].partitioner == "2,1"
    assert [p.var_name for p in by["emb:0"].part_config] == ["emb/part_0:0", "emb/part_1:0"]
    assert by["w1:0"].partitioner == "2,1" and by["b1:0"].partitioner == "2" and by["w2:0"].partitioner == "2,1"
    assert by["b2:0"].partitioner == "" and by["b2:0"].WhichOneof("synchronizer") == "PSSynchronizer"
    for p in by["emb:0"].part_config:
        assert p.PSSynchronizer.reduction_destination == "localhost:CPU:0"


def test_uneven_partitioned_ps(r0):
    s = UnevenPartitionedPS(local_proxy_variable=True).build(model(), r0)
    by = {n.var_name: n for n in s.node_config}
    assert by["emb:0"].partitioner == "3,1" and len(by["emb:0"].part_config) == 3
    assert by["w1:0"].partitioner == "3,1" and by["b1:0"].partitioner == "3" and by["w2:0"].partitioner == "3,1"
    assert by["b2:0"].partitioner == ""


def test_partitioned_ps_forced_gpu_shards(r0):
    s = PartitionedPS(num_shards=2, reduction_devices="gpu").build(model(), r0)
    emb = s.node_config[0]
    assert [p.PSSynchronizer.reduction_destination for p in emb.part_config] == ["localhost:GPU:0", "localhost:GPU:1"]


def test_all_reduce_groups(r0):
    s = AllReduce(chunk_size=2, compressor="HorovodCompressorEF").build(model(), r0)
    assert [n.AllReduceSynchronizer.group for n in s.node_config] == [0, 0, 1, 1, 2]
    assert all(n.AllReduceSynchronizer.compressor == 2 and n.AllReduceSynchronizer.spec == 1 for n in s.node_config)
    with pytest.raises(ValueError):
        AllReduce(chunk_size=0)
    s = AllReduce(compressor="PowerSGDCompressor", power_sgd_rank=2).build(model(), r0)
    assert s.node_config[0].AllReduceSynchronizer.compressor == 3
    assert s.node_config[0].AllReduceSynchronizer.power_sgd_rank == 2


def test_partitioned_ar(r0):
    s = PartitionedAR(chunk_size=3).build(model(), r0)
    by = {n.var_name: n for n in s.node_config}
    # counter advances by the number of shards: emb 0,1 | w1 2,3 | b1 4,5 | w2 6,7 | b2 8
    assert [p.AllReduceSynchronizer.group for p in by["emb:0"].part_config] == [0, 0]
    assert [p.AllReduceSynchronizer.group for p in by["w1:0"].part_config] == [0, 1]
    assert [p.AllReduceSynchronizer.group for p in by["w2:0"].part_config] == [2, 2]
    assert by["b2:0"].AllReduceSynchronizer.group == 2 and by["b2:0"].AllReduceSynchronizer.spec == 0


def test_random_axis(r0):
    seen = set()
    for seed in range(8):
        s = RandomAxisPartitionAR(chunk_size=4, seed=seed).build(model(), r0)
        by = {n.var_name: n for n in s.node_config}
        assert by["emb:0"].partitioner == "2,1"       # sparse: axis 0 only
        assert by["w2:0"].partitioner == "2,1"        # only axis 0 is wider than 1
        seen.add(by["w1:0"].partitioner)
    assert seen == {"2,1", "1,2"}


def test_parallax(r0):
    s = Parallax(chunk_size=2, local_proxy_variable=True).build(model(), r0)
    by = {n.var_name: n for n in s.node_config}
    assert by["emb:0"].WhichOneof("synchronizer") == "PSSynchronizer"
    assert not by["emb:0"].PSSynchronizer.local_replication        # sparse PS variables never get a proxy
    assert [by[v].AllReduceSynchronizer.group for v in ("w1:0", "b1:0", "w2:0", "b2:0")] == [0, 1, 1, 2]


def test_parallax_with_gpu_owners_row_shards_the_sparse_table(r0):
    """``reduction_devices="gpu"``: a row-sparse table becomes one row shard per GPU (each shard a parameter-server part on
    its GPU), dense variables keep their all-reduce groups, and a sparse variable inside control flow stays whole."""
    s = Parallax(chunk_size=2, reduction_devices="gpu").build(model(), r0)
    by = {n.var_name: n for n in s.node_config}
    emb = by["emb:0"]
    assert emb.partitioner == "2,1"                                     # axis 0 cut in two, axis 1 whole
    assert [p.var_name for p in emb.part_config] == ["emb/part_0:0", "emb/part_1:0"]
    owners = [p.PSSynchronizer.reduction_destination for p in emb.part_config]
    assert len(set(owners)) == 2 and all("GPU" in o.upper() for o in owners), owners
    assert all(p.PSSynchronizer.sync and not p.PSSynchronizer.local_replication for p in emb.part_config)
    assert [by[v].AllReduceSynchronizer.group for v in ("w1:0", "b1:0", "w2:0", "b2:0")] == [0, 1, 1, 2]
    f = torch.float32
    looped = FakeItem([VariableInfo("emb:0", (10000, 16), f, sparse_grad=True, in_control_flow=True), VariableInfo("w:0", (16, 16), f)])
    s2 = Parallax(chunk_size=2, reduction_devices="gpu").build(looped, r0)
    whole = {n.var_name: n for n in s2.node_config}["emb:0"]
    assert not whole.partitioner and whole.WhichOneof("synchronizer") == "PSSynchronizer"
