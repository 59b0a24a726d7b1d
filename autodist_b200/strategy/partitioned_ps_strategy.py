"""``PartitionedPS`` and ``UnevenPartitionedPS`` builders.

Reference: ``autodist/strategy/partitioned_ps_strategy.py:28-169`` and
``uneven_partition_ps_strategy.py:28-169``. Each variable is split along axis 0
into the smallest divisor >= 2 of its first dimension (or, for the uneven
variant, the smallest number that does NOT divide it) and the shards are placed
on the least-loaded reduction devices, round-robin when shards outnumber them.

Additions for one NVSwitch box: ``num_shards`` forces a shard count (e.g. the
number of GPUs) and ``reduction_devices="gpu"`` makes GPUs the shard owners, so
that a variable's gradient is reduce-scattered to its owners and updated there.
"""
from autodist_b200.const import ENV
from autodist_b200.strategy import _placement as P
from autodist_b200.strategy.base import StrategyBuilder


class PartitionedPS(StrategyBuilder):
    _shard_rule = staticmethod(P.min_divisor_shards)

    def __init__(self, local_proxy_variable=False, sync=True, staleness=0, num_shards=None,
                 reduction_devices="cpu"):
        if staleness > 0 and not sync:
            raise AssertionError("If staleness is positive, sync has to be set True.")
        self._local_proxy_variable = local_proxy_variable
        self._sync = sync
        self._staleness = staleness
        self._forced_shards = num_shards
        self._placement = reduction_devices
        self.loads = {}

    def get_num_shards(self, var):
        if len(var.shape) == 0:
            return 1
        n = int(var.shape[0])
        if self._forced_shards is not None:
            return max(1, min(int(self._forced_shards), n))
        return self._shard_rule(n)

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        self._greedy = P.GreedyLoads(P.reduction_devices(resource_spec, self._placement))
        self.loads = self._greedy.loads
        s.node_config.extend(self._gen_ps_node_config(v) for v in graph_item.trainable_var_op_to_var.values())
        return s

    def _gen_ps_node_config(self, var):
        # The reference keeps partitioning even with a single server (its guard is
        # `len(loads) < 1`), and never partitions a variable consumed by control flow.
        if (len(self._greedy) < 1 and not ENV.AUTODIST_IS_TESTING.val) or var.in_control_flow:
            num_shards = 1
        else:
            num_shards = self.get_num_shards(var)
        owners = self._greedy.least_loaded(num_shards)
        for dev in owners:
            self._greedy.add(dev, P.byte_size_load_fn(var) / num_shards)
        args = (self._local_proxy_variable, self._sync, self._staleness)
        if num_shards == 1:
            return P.ps_node(var.name, owners[0], *args)
        node = P.strategy_pb2.Strategy.Node()
        node.var_name = var.name
        node.partitioner = P.partition_string(len(var.shape), 0, min(num_shards, int(var.shape[0])))
        for i in range(num_shards):
            P.fill_ps(node.part_config.add(var_name=P.part_name(var.name, i)), owners[i], *args)
        return node


class UnevenPartitionedPS(PartitionedPS):
    """Same placement, but a shard count that does not divide dim 0 (exercises uneven splits)."""
    _shard_rule = staticmethod(P.first_non_divisor_shards)
