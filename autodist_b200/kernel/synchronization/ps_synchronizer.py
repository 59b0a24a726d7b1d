"""Parameter-server synchronizer.

Capability parity with ``autodist/kernel/synchronization/ps_synchronizer.py:44-761``:
each variable (or shard) has one owner device, replicas push gradients to it, the
owner applies the averaged gradient and replicas read the result; ``sync`` and
``staleness`` select a fully synchronous step, a bounded-staleness gate or no
gate at all; ``local_replication`` keeps a local mirror that is refreshed right
after the update instead of being pulled before the next read.

On one NVSwitch box the owner is a GPU rank: the push is a reduce(-scatter) to
the owner, the update runs on the owner's shard and the refresh is an
all-gather. The accumulator / token-queue machinery of the reference becomes
the collective itself (synchronous mode) or an epoch counter per rank with a
bounded wait (``staleness`` > 0).
"""
from autodist_b200.kernel.device.resolver import DeviceResolver
from autodist_b200.kernel.synchronization.synchronizer import Synchronizer, VarPart
from autodist_b200.proto import synchronizers_pb2


class PSSynchronizer(Synchronizer):
    def __init__(self, config: synchronizers_pb2.PSSynchronizer):
        super().__init__()
        self.target_device = config.reduction_destination
        self._local_replication = config.local_replication
        self._sync = config.sync
        self._staleness = config.staleness
        if self._staleness > 0 and not self._sync:
            raise ValueError("If staleness is positive, sync has to be set true.")

    @property
    def owner_rank(self):
        return DeviceResolver.rank_of(self.target_device)

    def in_graph_apply(self, plan, part: VarPart):
        """Node-local part: replicas of a node average their gradients before anything leaves the node."""
        plan.add_ps(part, owner=self.owner_rank, local_replication=self._local_replication,
                    sync=self._sync, staleness=self._staleness)

    def between_graph_apply(self, plan, part: VarPart):
        """Cross-worker part: pick the gate that orders updates against the next step's reads."""
        if not self._sync:
            plan.set_ps_gate(part, "async")
        elif self._staleness > 0:
            plan.set_ps_gate(part, "stale", self._staleness)
        else:
            plan.set_ps_gate(part, "sync")
