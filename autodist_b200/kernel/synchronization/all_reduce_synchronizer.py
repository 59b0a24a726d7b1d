"""All-reduce synchronizer: mean of a gradient over every replica.

Capability parity with ``autodist/kernel/synchronization/all_reduce_synchronizer.py:38-201``.
Variables of one ``group`` share a bucket (the reference relies on TensorFlow's
scoped allocator to merge same-group collectives); dense gradients go through
the bucket's compressor; row-sparse gradients are exchanged as (indices, values)
and, unlike the reference (which concatenates without dividing,
``all_reduce_synchronizer.py:155-169``), averaged, so that a variable trains the
same under all-reduce and under a parameter server.
"""
from autodist_b200.kernel.synchronization.collective_key import get_collective_keys
from autodist_b200.kernel.synchronization.synchronizer import Synchronizer, VarPart
from autodist_b200.proto import synchronizers_pb2
from autodist_b200.utils import logging


class AllReduceSynchronizer(Synchronizer):
    def __init__(self, config: synchronizers_pb2.AllReduceSynchronizer):
        super().__init__()
        self._spec = synchronizers_pb2.AllReduceSynchronizer.Spec.Name(config.spec)
        self._compressor_type = synchronizers_pb2.AllReduceSynchronizer.Compressor.Name(config.compressor)
        self._group = config.group
        self._power_sgd_rank = config.power_sgd_rank or 1

    @property
    def group(self):
        return self._group

    @property
    def compressor_type(self):
        return self._compressor_type

    def in_graph_apply(self, plan, part: VarPart):
        if self.num_replicas * self.num_workers <= 1:
            return  # nothing to synchronise with
        keys = get_collective_keys()
        group_key = keys.generate_group_key(self.all_canonical_replica_devices)
        instance_key = keys.generate_instance_key(part.part_name)
        if part.sparse:
            if self._compressor_type != "NoneCompressor":
                logging.warning("compressor %s is not applied to the sparse gradient of %s",
                                self._compressor_type, part.part_name)
            plan.add_sparse_all_reduce(part, group_key, instance_key)
        else:
            plan.add_all_reduce(part, self._group, self._compressor_type, self._spec,
                                self._power_sgd_rank, group_key, instance_key)

    def between_graph_apply(self, plan, part: VarPart):
        """The bucket's collective already spans every replica of every node."""
        return
