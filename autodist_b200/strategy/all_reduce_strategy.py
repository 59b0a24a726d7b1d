"""``AllReduce``, ``PartitionedAR`` and ``RandomAxisPartitionAR`` builders.

Reference: ``autodist/strategy/all_reduce_strategy.py:28-90``,
``partitioned_all_reduce_strategy.py:28-130`` and
``random_axis_partition_all_reduce_strategy.py:28-141``. ``chunk_size`` counts
*variables* merged into one collective group (group = index // chunk_size).
"""
import numpy as np

from autodist_b200.strategy import _placement as P
from autodist_b200.strategy.base import StrategyBuilder

_COMPRESSORS = ("NoneCompressor", "HorovodCompressor", "HorovodCompressorEF", "PowerSGDCompressor")
_SPECS = ("AUTO", "NCCL", "RING")


class AllReduce(StrategyBuilder):
    def __init__(self, chunk_size=128, all_reduce_spec="NCCL", compressor="NoneCompressor", power_sgd_rank=1):
        if chunk_size < 1:
            raise ValueError("The chunk_size must be greater than zero.")
        if compressor not in _COMPRESSORS:
            raise ValueError(f"unknown compressor {compressor!r}; choose from {_COMPRESSORS}")
        if all_reduce_spec not in _SPECS:
            raise ValueError(f"unknown all_reduce_spec {all_reduce_spec!r}; choose from {_SPECS}")
        self.chunk_size = chunk_size
        self.all_reduce_spec = all_reduce_spec
        self.compressor = compressor
        self.power_sgd_rank = power_sgd_rank if compressor == "PowerSGDCompressor" else 0

    def _gen_all_reduce_node_config(self, var_name, group=0, all_reduce_spec=None, compressor=None):
        return P.all_reduce_node(var_name, group, all_reduce_spec or self.all_reduce_spec,
                                 compressor or self.compressor, self.power_sgd_rank)

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        for i, var in enumerate(graph_item.trainable_var_op_to_var.values()):
            s.node_config.append(self._gen_all_reduce_node_config(var.name, group=i // self.chunk_size))
        return s


class PartitionedAR(StrategyBuilder):
    """Split every variable on axis 0 and all-reduce the pieces as separate messages."""

    def __init__(self, chunk_size=128):
        if chunk_size < 1:
            raise ValueError("The chunk_size must be greater than zero.")
        self.chunk_size = chunk_size

    def get_num_shards_and_axis(self, var):
        if len(var.shape) == 0:
            return 1, 0
        return P.min_divisor_shards(int(var.shape[0])), 0

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        counter = 0
        for var in graph_item.trainable_var_op_to_var.values():
            # a variable read inside data-dependent control flow stays whole (as in the partitioned PS builders)
            num_shards, axis = (1, 0) if var.in_control_flow else self.get_num_shards_and_axis(var)
            node = s.node_config.add(var_name=var.name)
            if num_shards <= 1:
                P.fill_all_reduce(node, counter // self.chunk_size, "AUTO")
            else:
                node.partitioner = P.partition_string(len(var.shape), axis, num_shards)
                for i in range(num_shards):
                    P.fill_all_reduce(node.part_config.add(var_name=P.part_name(var.name, i)),
                                      (counter + i) // self.chunk_size, "AUTO")
            counter += num_shards
        return s


class RandomAxisPartitionAR(PartitionedAR):
    """As ``PartitionedAR`` with the axis drawn uniformly among dims > 1 (axis 0 for sparse gradients)."""

    def __init__(self, chunk_size=128, seed=None):
        super().__init__(chunk_size)
        self._rng = np.random.RandomState(seed) if seed is not None else np.random

    def get_num_shards_and_axis(self, var):
        wide = [i for i, d in enumerate(var.shape) if d > 1]
        if not wide:
            return 1, 0
        axis = 0 if var.sparse_grad else wide[int(self._rng.randint(0, len(wide)))]
        return P.min_divisor_shards(int(var.shape[axis])), axis
