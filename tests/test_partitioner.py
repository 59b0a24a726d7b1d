"""Shard plans: sizes, offsets, sparse routing and re-merging (property style, prime / uneven / axis != 0)."""
import pytest
import torch

from autodist_b200.kernel.partitioner import (PartitionerConfig, make_shard_plan, shard_of_rows, split_sizes)


def test_config_parsing():
    pc = PartitionerConfig(partition_str="1,4,1")
    assert pc.axis == 1 and pc.num_shards == 4 and pc.partition_list == [1, 4, 1]
    assert PartitionerConfig(partition_list=[2, 1]).partition_str == "2,1"
    for bad in ("2,2", "0,1", "", "a,b"):
        with pytest.raises(ValueError):
            PartitionerConfig(partition_str=bad)


@pytest.mark.parametrize("n", [1, 2, 3, 7, 16, 97, 1000, 30522])
@pytest.mark.parametrize("k", [1, 2, 3, 4, 7, 8])
def test_split_sizes_and_row_routing(n, k):
    k = min(k, n)
    sizes = split_sizes(n, k)
    assert sum(sizes) == n and max(sizes) - min(sizes) <= 1 and sorted(sizes, reverse=True) == sizes
    ids = torch.arange(n)
    owner = shard_of_rows(ids, n, k)
    expect = torch.repeat_interleave(torch.arange(k), torch.tensor(sizes))
    assert torch.equal(owner, expect)


@pytest.mark.parametrize("shape,pstr", [((10, 4), "3,1"), ((10, 4), "1,2"), ((7,), "7"), ((5, 3, 4), "1,1,3")])
def test_dense_split_and_merge(shape, pstr):
    plan = make_shard_plan("v:0", shape, pstr)
    t = torch.arange(float(torch.tensor(shape).prod())).view(shape)
    merged = torch.zeros_like(t)
    for i, piece in enumerate(plan.split_dense(t)):
        plan.view(merged, i).copy_(piece)
        name, full, off, shp = plan.save_slice_info(i)
        assert name == "v:0" and full == list(shape) and list(piece.shape) == shp
    assert torch.equal(merged, t)
    assert plan.part_names[0] == "v/part_0:0"


def test_sparse_split():
    plan = make_shard_plan("emb:0", (10, 2), "3,1")   # sizes 4,3,3
    idx = torch.tensor([0, 3, 4, 9, 6, 4])
    val = torch.arange(12.0).view(6, 2)
    parts = plan.split_sparse(idx, val)
    assert [p[0].tolist() for p in parts] == [[0, 3], [0, 2, 0], [2]]
    dense = torch.zeros(10, 2).index_add_(0, idx, val)
    rebuilt = torch.zeros(10, 2)
    for i, (li, lv) in enumerate(parts):
        plan.view(rebuilt, i).index_add_(0, li, lv)
    assert torch.equal(dense, rebuilt)
