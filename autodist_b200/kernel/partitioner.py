"""Variable partitioning: from ``"1,4,1"`` strings to shard plans, split gradients and row routing.

Capability parity with ``autodist/kernel/partitioner.py:32-714``. The reference
rewrites the TensorFlow graph (new ``PartitionedVariable``, sliced gradients,
re-run ``apply_gradients``, rebuilt savers); here a variable keeps its full
tensor on every replica and a ``ShardPlan`` says which contiguous slice of which
axis each shard covers. The runtime hands shard views to the owner's optimizer
and the saver writes shards back at their offsets, so checkpoints hold one tensor
under the original name.
"""
from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from autodist_b200.kernel.kernel import Kernel
from autodist_b200.utils import logging


class PartitionerConfig:
    """Parsed partition string: exactly one axis may have more than one shard."""

    def __init__(self, partition_list=None, partition_str=None):
        if (partition_list is None) == (partition_str is None):
            raise ValueError("give exactly one of partition_list / partition_str")
        if partition_str is not None:
            try:
                partition_list = [int(x) for x in partition_str.split(",") if x.strip() != ""]
            except ValueError as e:
                raise ValueError(f"malformed partition string {partition_str!r}") from e
        partition_list = [int(x) for x in partition_list]
        if not partition_list:
            raise ValueError("empty partition list")
        if any(x < 1 for x in partition_list):
            raise ValueError(f"partition counts must be positive: {partition_list}")
        if sum(1 for x in partition_list if x > 1) > 1:
            raise ValueError(f"only one axis may be partitioned: {partition_list}")
        self._list = partition_list

    @property
    def partition_list(self):
        return list(self._list)

    @property
    def partition_str(self):
        return ",".join(str(x) for x in self._list)

    @property
    def num_shards(self):
        return max(self._list)

    @property
    def axis(self):
        for i, x in enumerate(self._list):
            if x > 1:
                return i
        return 0


def split_sizes(n, k):
    """Sizes of ``k`` contiguous shards of a dimension of ``n``: the first ``n % k`` get one extra."""
    q, r = divmod(n, k)
    return [q + (1 if i < r else 0) for i in range(k)]


def shard_of_rows(ids, n, k):
    """Shard index of each row id under ``split_sizes(n, k)``: ``max(id // (q+1), (id - r) // q)``."""
    q, r = divmod(n, k)
    if q == 0:
        return ids.clone()
    return torch.maximum(torch.div(ids, q + 1, rounding_mode="floor"),
                         torch.div(ids - r, q, rounding_mode="floor"))


@dataclass
class ShardPlan:
    var_name: str
    shape: Tuple[int, ...]
    axis: int
    sizes: List[int]
    offsets: List[int]
    part_names: List[str]

    @property
    def num_shards(self):
        return len(self.sizes)

    def slice_of(self, i):
        return self.axis, self.offsets[i], self.sizes[i]

    def view(self, tensor, i):
        """Shard ``i`` of ``tensor`` (shaped like the variable) as a view."""
        return tensor.narrow(self.axis, self.offsets[i], self.sizes[i])

    def split_dense(self, grad):
        return [self.view(grad, i) for i in range(self.num_shards)]

    def split_sparse(self, indices, values):
        """Route row-sparse ``(indices, values)`` to shards; returned indices are shard-local."""
        assert self.axis == 0, "sparse gradients are only partitioned along axis 0"
        owner = shard_of_rows(indices, self.shape[0], self.num_shards)
        out = []
        for i in range(self.num_shards):
            mask = owner == i
            out.append((indices[mask] - self.offsets[i], values[mask]))
        return out

    def save_slice_info(self, i):
        """(full_name, full_shape, var_offset, var_shape) of shard ``i`` for the checkpoint writer."""
        off = [0] * len(self.shape)
        shp = list(self.shape)
        off[self.axis] = self.offsets[i]
        shp[self.axis] = self.sizes[i]
        return self.var_name, list(self.shape), off, shp


def make_shard_plan(var_name, shape, partition_str, part_names=None):
    pc = PartitionerConfig(partition_str=partition_str)
    if len(pc.partition_list) != len(shape):
        raise ValueError(f"partitioner {partition_str!r} does not match rank of {var_name} {tuple(shape)}")
    axis, k = pc.axis, pc.num_shards
    k = min(k, int(shape[axis])) if len(shape) else 1
    sizes = split_sizes(int(shape[axis]), k)
    offsets = [sum(sizes[:i]) for i in range(k)]
    op_name = var_name[:-2] if var_name.endswith(":0") else var_name
    names = list(part_names) if part_names else [f"{op_name}/part_{i}:0" for i in range(k)]
    return ShardPlan(var_name, tuple(int(d) for d in shape), axis, sizes, offsets, names[:k])


class VariablePartitioner(Kernel):
    """Pass 1 of the transformer: one ``ShardPlan`` per strategy node that carries a partitioner."""

    def __init__(self, key, node_config, graph_item):
        super().__init__(key)
        self.node_config = node_config
        self.graph_item = graph_item

    def _apply(self) -> Dict[str, ShardPlan]:
        plans = {}
        variables = self.graph_item.variables
        for node in self.node_config:
            if not node.partitioner:
                continue
            var = variables[node.var_name]
            if var.in_control_flow:
                raise ValueError(f"{var.name} is consumed by control flow and cannot be partitioned")
            plan = make_shard_plan(var.name, var.shape, node.partitioner, [p.var_name for p in node.part_config])
            if var.sparse_grad and plan.axis != 0:
                raise ValueError(f"{var.name} has sparse gradients: it can only be partitioned along axis 0")
            if plan.num_shards != len(node.part_config):
                logging.warning("%s: %d part configs for %d shards", var.name, len(node.part_config), plan.num_shards)
            # The strategy's part names become the actual shard names.
            for i, part in enumerate(node.part_config[:plan.num_shards]):
                part.var_name = plan.part_names[i]
            plans[var.name] = plan
        return plans
