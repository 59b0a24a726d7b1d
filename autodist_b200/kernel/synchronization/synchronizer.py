"""Synchronizer interface.

A synchronizer owns the rule by which one variable (or one shard of it) turns
per-replica gradients into one update. Capability parity with
``autodist/kernel/synchronization/synchronizer.py:28-118``; instead of rewriting
a TensorFlow graph in two phases, the two phases register work in a
``DistributedPlan``:

* ``in_graph_apply``  - aggregation among the replicas of one node,
* ``between_graph_apply`` - aggregation across nodes / the update gate.

With one process per device inside one ``torch.distributed`` job both phases
end up in the same collective; they stay separate calls so that a strategy that
distinguishes node-local from cross-node behaviour (``sync``, ``staleness``)
has a place to say so.
"""
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Optional


@dataclass
class VarPart:
    """One synchronised unit: a whole variable or one shard of it."""
    var_name: str
    part_name: str
    part_index: Optional[int]
    axis: int
    offset: int
    size: int               # extent along ``axis``; -1 = whole variable
    sparse: bool
    numel: int

    def view(self, tensor):
        if self.part_index is None:
            return tensor
        return tensor.narrow(self.axis, self.offset, self.size)


class Synchronizer(ABC):
    def __init__(self):
        self.num_workers = 1
        self.num_replicas = 1
        self.worker_device = None
        self.worker_id = 0
        self.all_canonical_replica_devices = []
        self.is_chief = True
        self.var_op_to_agg_grad = None

    def assign_cluster_information(self, num_workers, num_replicas, worker_device, worker_id,
                                   canonical_replica_devices, is_chief=False):
        self.num_workers = num_workers
        self.num_replicas = num_replicas
        self.worker_device = worker_device
        self.worker_id = worker_id
        self.all_canonical_replica_devices = list(canonical_replica_devices)
        self.is_chief = is_chief
        return self

    @abstractmethod
    def in_graph_apply(self, plan, part: VarPart):
        """Register the node-local aggregation of ``part`` in ``plan``."""

    @abstractmethod
    def between_graph_apply(self, plan, part: VarPart):
        """Register the cross-node aggregation / gate of ``part`` in ``plan``."""

    @classmethod
    def create(cls, name, *args, **kwargs):
        """Instantiate the subclass called ``name`` (the proto's ``oneof`` field name)."""
        from autodist_b200.kernel.synchronization import all_reduce_synchronizer, ps_synchronizer  # noqa: F401
        for sub in cls.__subclasses__():
            if sub.__name__ == name:
                return sub(*args, **kwargs)
        raise ValueError(f"{name} is not a valid synchronizer name")
