"""Transformer: (captured graph, compiled strategy) -> ``DistributedPlan``.

Same pass order as ``autodist/kernel/graph_transformer.py:55-92``: partition
variables, create one synchronizer per variable or shard, replicate, apply the
node-local phase of every synchronizer, then the cross-node phase. A text dump
of the plan is kept after each stage (the reference writes TensorBoard graph
files ``0-original`` ... ``3-transformed``).
"""
from autodist_b200.kernel.partitioner import VariablePartitioner
from autodist_b200.kernel.plan import DistributedPlan
from autodist_b200.kernel.replicator import Replicator
from autodist_b200.kernel.synchronization.synchronizer import Synchronizer, VarPart
from autodist_b200.utils import logging, visualization_util


class GraphTransformer:
    def __init__(self, compiled_strategy, cluster, graph_item, rank=0):
        self._strategy = compiled_strategy
        self._cluster = cluster
        self.graph_item = graph_item
        self._rank = rank
        self.num_local_replicas = 0

    def _parts_of(self, node, shard_plans):
        var = self.graph_item.variables[node.var_name]
        if node.partitioner and node.var_name in shard_plans:
            sp = shard_plans[node.var_name]
            out = []
            for i, part_node in enumerate(node.part_config[:sp.num_shards]):
                shape = list(var.shape)
                shape[sp.axis] = sp.sizes[i]
                numel = 1
                for d in shape:
                    numel *= d
                out.append((part_node, VarPart(var.name, sp.part_names[i], i, sp.axis, sp.offsets[i],
                                               sp.sizes[i], var.sparse_grad, numel)))
            return out
        return [(node, VarPart(var.name, var.name, None, 0, 0, -1, var.sparse_grad, var.numel))]

    def _initialize_synchronizers(self, shard_plans, replica):
        out = []
        for node in self._strategy.node_config:
            for cfg_node, part in self._parts_of(node, shard_plans):
                which = cfg_node.WhichOneof("synchronizer")
                if which is None:
                    raise ValueError(f"strategy node {cfg_node.var_name} has no synchronizer")
                sync = Synchronizer.create(which, getattr(cfg_node, which))
                sync.assign_cluster_information(
                    num_workers=replica.num_workers, num_replicas=replica.num_local_replicas,
                    worker_device=replica.device, worker_id=replica.rank,
                    canonical_replica_devices=replica.replicas, is_chief=replica.rank == 0)
                out.append((sync, part))
        return out

    def transform(self):
        item = self.graph_item
        logging.debug("Transforming the original graph to a distributed plan...")
        visualization_util.log_graph(item.graph_text(), "0-original")
        if getattr(item, "tracer", None) is not None and getattr(item.tracer, "graph", None) is not None:
            visualization_util.log_fx_graph(item.tracer.graph, "0-original")

        shard_plans = VariablePartitioner.apply(self._strategy.node_config, item)
        visualization_util.log_graph(
            "\n".join(f"{n}: axis {p.axis} sizes {p.sizes}" for n, p in shard_plans.items()), "1-after-partition")

        replica = Replicator.apply(list(self._strategy.graph_config.replicas), self._rank)
        self.num_local_replicas = replica.num_local_replicas
        plan = DistributedPlan(replica, shard_plans, {n: v.shape for n, v in item.variables.items()})
        synchronizers = self._initialize_synchronizers(shard_plans, replica)

        for sync, part in synchronizers:
            sync.in_graph_apply(plan, part)
        visualization_util.log_graph(plan.describe(), "2-after-in-graph")
        for sync, part in synchronizers:
            sync.between_graph_apply(plan, part)
        visualization_util.log_graph(plan.describe(), "3-transformed")
        logging.debug("Successfully built the distributed plan.")
        return plan
