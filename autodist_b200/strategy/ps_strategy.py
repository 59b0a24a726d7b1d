"""``PS`` and ``PSLoadBalancing`` builders.

Reference: ``autodist/strategy/ps_strategy.py:28-76`` (every variable on the
first CPU device) and ``ps_lb_strategy.py:28-117`` (greedy byte-load balancing,
the framework's default builder).
"""
from autodist_b200.strategy import _placement as P
from autodist_b200.strategy.base import StrategyBuilder


class _PSBase(StrategyBuilder):
    def __init__(self, local_proxy_variable=False, sync=True, staleness=0, reduction_devices="cpu"):
        if staleness > 0 and not sync:
            raise AssertionError("If staleness is positive, sync has to be set true.")
        self._local_proxy_variable = local_proxy_variable
        self._sync = sync
        self._staleness = staleness
        self._placement = reduction_devices
        self.loads = {}


class PS(_PSBase):
    """All variables synchronised through one parameter server (the first reduction device)."""

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        dest = P.reduction_devices(resource_spec, self._placement)[0]
        s.node_config.extend(
            P.ps_node(v.name, dest, self._local_proxy_variable, self._sync, self._staleness)
            for v in graph_item.trainable_var_op_to_var.values())
        return s


class PSLoadBalancing(_PSBase):
    """Each variable goes to the reduction device with the least accumulated bytes."""

    def _begin(self, resource_spec):
        self._greedy = P.GreedyLoads(P.reduction_devices(resource_spec, self._placement))
        self.loads = self._greedy.loads

    def _gen_ps_node_config(self, var, local_proxy_variable, sync, staleness):
        dest = self._greedy.least_loaded(1)[0]
        self._greedy.add(dest, P.byte_size_load_fn(var))
        return P.ps_node(var.name, dest, local_proxy_variable, sync, staleness)

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        self._begin(resource_spec)
        s.node_config.extend(
            self._gen_ps_node_config(v, self._local_proxy_variable, self._sync, self._staleness)
            for v in graph_item.trainable_var_op_to_var.values())
        return s
