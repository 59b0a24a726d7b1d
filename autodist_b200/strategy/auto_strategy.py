"""``AutoStrategy``: build every candidate strategy, predict its step time with the simulator, return the best.

The reference names this capability (``network_bandwidth`` exists "for AutoStrategy",
``autodist/resource_spec.py:209-215``) but its snapshot ships no implementation.
"""
from autodist_b200.strategy.all_reduce_strategy import AllReduce, PartitionedAR
from autodist_b200.strategy.base import StrategyBuilder
from autodist_b200.strategy.parallax_strategy import Parallax
from autodist_b200.strategy.partitioned_ps_strategy import PartitionedPS
from autodist_b200.strategy.ps_strategy import PS, PSLoadBalancing


class AutoStrategy(StrategyBuilder):
    def __init__(self, candidates=None, compute_ms=0.0):
        self._candidates = candidates
        self._compute_ms = compute_ms
        self.ranking = []

    def _default_candidates(self, resource_spec):
        n = max(2, len(resource_spec.replica_devices))
        return {
            "PS": PS(reduction_devices="gpu"),
            "PSLoadBalancing": PSLoadBalancing(reduction_devices="gpu"),
            "PartitionedPS": PartitionedPS(num_shards=n, reduction_devices="gpu"),
            "AllReduce": AllReduce(chunk_size=256),
            "AllReduce_fp16_EF": AllReduce(chunk_size=256, compressor="HorovodCompressorEF"),
            "PartitionedAR": PartitionedAR(chunk_size=256),
            "Parallax": Parallax(chunk_size=256, reduction_devices="gpu"),
        }

    def build(self, graph_item, resource_spec):
        from autodist_b200.simulator.simulator import rank_strategies
        cands = self._candidates or self._default_candidates(resource_spec)
        self.ranking = rank_strategies(cands, graph_item, resource_spec, self._compute_ms)
        return self.ranking[0][2]
