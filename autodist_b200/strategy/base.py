"""Strategy wrapper, builder interface and compiler.

Capability parity with the reference's ``autodist/strategy/base.py:28-168``:
a ``Strategy`` wraps the protobuf message, gets a UTC-timestamp id, and is
written to ``<working dir>/strategies/<id>`` so that every rank loads the
chief's decision; ``StrategyCompiler`` prunes nodes without an update and
resolves device strings through a pluggable resolver.
"""
import datetime
import os
from abc import ABC, abstractmethod

from autodist_b200 import const
from autodist_b200.proto import strategy_pb2


class Strategy:
    """In-memory handle of one ``autodist.proto.Strategy`` message."""

    def __init__(self, strategy=None):
        self._strategy = strategy if strategy is not None else strategy_pb2.Strategy()
        if strategy is None:
            self._strategy.id = datetime.datetime.now(datetime.timezone.utc).strftime("%Y%m%dT%H%M%SM%f")

    # -- message access ---------------------------------------------------
    @property
    def id(self):
        return self._strategy.id

    @property
    def path(self):
        return self._strategy.path

    @property
    def node_config(self):
        return self._strategy.node_config

    @node_config.setter
    def node_config(self, value):
        del self._strategy.node_config[:]
        self._strategy.node_config.extend(value)

    @property
    def graph_config(self):
        return self._strategy.graph_config

    @property
    def proto(self):
        return self._strategy

    def copy(self):
        other = strategy_pb2.Strategy()
        other.CopyFrom(self._strategy)
        return Strategy(strategy=other)

    def __str__(self):
        return str(self._strategy)

    def __eq__(self, other):
        return isinstance(other, Strategy) and self._strategy == other._strategy

    # -- persistence ----------------------------------------------------------
    def serialize(self, path=None):
        if path is None:
            os.makedirs(const.DEFAULT_SERIALIZATION_DIR, exist_ok=True)
            path = os.path.join(const.DEFAULT_SERIALIZATION_DIR, self.id)
        self._strategy.path = path
        tmp = f"{path}.{os.getpid()}.tmp"
        with open(tmp, "wb") as f:
            f.write(self._strategy.SerializeToString())
        os.replace(tmp, path)  # ranks polling for the file never see a half-written one
        return path

    @classmethod
    def deserialize(cls, strategy_id=None, path=None):
        if path is None:
            assert strategy_id is not None, "need a strategy id or a path"
            path = os.path.join(const.DEFAULT_SERIALIZATION_DIR, strategy_id)
        msg = strategy_pb2.Strategy()
        with open(path, "rb") as f:
            msg.ParseFromString(f.read())
        return cls(strategy=msg)


class StrategyBuilder(ABC):
    """Maps ``(graph_item, resource_spec)`` to a ``Strategy``."""

    @abstractmethod
    def build(self, graph_item, resource_spec):
        raise NotImplementedError

    @staticmethod
    def _new_strategy(resource_spec):
        """A strategy whose replica list is every GPU plus the CPUs of GPU-less nodes."""
        s = Strategy()
        gpu_nodes = resource_spec.node_gpu_devices
        s.graph_config.replicas.extend(k for k, _ in resource_spec.gpu_devices)
        for host, cpus in resource_spec.node_cpu_devices.items():
            if host not in gpu_nodes:
                s.graph_config.replicas.extend(cpus)
        return s


class StrategyCompiler:
    """Makes a builder's output executable for one captured graph.

    1. drops nodes of variables that receive no update (no gradient),
    2. rewrites every device string through ``device_resolver``.
    """

    def __init__(self, graph_item):
        self._graph_item = graph_item
        self._device_resolver = None

    def set_device_resolver(self, resolver):
        self._device_resolver = resolver
        return self

    def _resolve_node(self, node):
        which = node.WhichOneof("synchronizer")
        if which == "PSSynchronizer" and node.PSSynchronizer.reduction_destination:
            node.PSSynchronizer.reduction_destination = self._device_resolver(
                node.PSSynchronizer.reduction_destination)
        for part in node.part_config:
            self._resolve_node(part)

    def compile(self, strategy):
        strategy = strategy.copy()
        updated = self._graph_item.updated_variable_names()
        strategy.node_config = [n for n in strategy.node_config if n.var_name in updated]
        if self._device_resolver is not None:
            for node in strategy.node_config:
                self._resolve_node(node)
            resolved = [self._device_resolver(r) for r in strategy.graph_config.replicas]
            del strategy.graph_config.replicas[:]
            strategy.graph_config.replicas.extend(resolved)
        return strategy
