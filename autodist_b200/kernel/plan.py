"""The executable result of the transformer passes.

Where the reference's transformer emits a rewritten ``tf.Graph``
(``autodist/kernel/graph_transformer.py:55-92``), this framework emits a
``DistributedPlan``: which replica this process is, how variables are sharded,
which gradient parts share an all-reduce bucket (and its compressor), and which
parts are pushed to which owner rank under which gate. The step engine
executes the plan around the captured forward/backward.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from autodist_b200.kernel.synchronization.synchronizer import VarPart


@dataclass
class ARBucket:
    group: int
    compressor_type: str
    spec: str
    power_sgd_rank: int
    group_key: int
    parts: List[VarPart] = field(default_factory=list)
    instance_keys: List[int] = field(default_factory=list)
    shapes: List[Tuple[int, ...]] = field(default_factory=list)

    @property
    def key(self):
        return (self.group, self.compressor_type, self.spec)

    @property
    def numel(self):
        return sum(p.numel for p in self.parts)

    def member_shapes(self):
        return list(self.shapes)


@dataclass
class PSEntry:
    part: VarPart
    owner: int
    local_replication: bool
    sync: bool
    staleness: int
    gate: str = "sync"       # "sync" | "stale" | "async"


@dataclass
class ReplicaInfo:
    """Pass 2 (replication) result: which replica this process runs and who its node-mates are."""
    rank: int
    world_size: int
    device: str                      # replica device string of this rank
    replicas: List[str]              # all replica device strings in rank order
    local_ranks: List[int]           # ranks on this rank's node, in device order
    num_workers: int                 # number of nodes

    @property
    def local_replica_index(self):
        return self.local_ranks.index(self.rank)

    @property
    def num_local_replicas(self):
        return len(self.local_ranks)


class DistributedPlan:
    def __init__(self, replica: ReplicaInfo, shard_plans, var_shapes):
        self.replica = replica
        self.shard_plans = shard_plans            # var name -> ShardPlan
        self.var_shapes = var_shapes              # var name -> shape
        self.ar_buckets: Dict[tuple, ARBucket] = {}
        self.sparse_all_reduce: List[Tuple[VarPart, int, int]] = []
        self.ps_entries: Dict[str, PSEntry] = {}
        self.stages: List[Tuple[str, str]] = []   # (stage name, text dump) for visualisation

    # -- registration calls made by synchronizers ---------------------------
    def _part_shape(self, part):
        shape = list(self.var_shapes[part.var_name])
        if part.part_index is not None:
            shape[part.axis] = part.size
        return tuple(shape)

    def add_all_reduce(self, part, group, compressor_type, spec, power_sgd_rank, group_key, instance_key):
        key = (group, compressor_type, spec)
        b = self.ar_buckets.get(key)
        if b is None:
            b = self.ar_buckets[key] = ARBucket(group, compressor_type, spec, power_sgd_rank, group_key)
        b.parts.append(part)
        b.instance_keys.append(instance_key)
        b.shapes.append(self._part_shape(part))

    def add_sparse_all_reduce(self, part, group_key, instance_key):
        self.sparse_all_reduce.append((part, group_key, instance_key))

    def add_ps(self, part, owner, local_replication, sync, staleness):
        self.ps_entries[part.part_name] = PSEntry(part, owner, local_replication, sync, staleness)

    def set_ps_gate(self, part, gate, staleness=0):
        e = self.ps_entries[part.part_name]
        e.gate = gate
        if gate == "stale":
            e.staleness = staleness

    # -- queries ------------------------------------------------------------------
    def ordered_buckets(self):
        return [self.ar_buckets[k] for k in sorted(self.ar_buckets)]

    def ps_by_owner(self):
        out: Dict[int, List[PSEntry]] = {}
        for e in self.ps_entries.values():
            out.setdefault(e.owner, []).append(e)
        return out

    @property
    def gate_mode(self):
        modes = {e.gate for e in self.ps_entries.values()}
        if "async" in modes:
            return "async"
        if "stale" in modes:
            return "stale"
        return "sync"

    @property
    def staleness(self):
        return max([e.staleness for e in self.ps_entries.values() if e.gate == "stale"] or [0])

    def describe(self):
        lines = [f"replica {self.replica.rank}/{self.replica.world_size} on {self.replica.device}"]
        for b in self.ordered_buckets():
            lines.append(f"all-reduce group {b.group} [{b.compressor_type}/{b.spec}] key {b.group_key} "
                         f"{len(b.parts)} parts, {b.numel} elements")
        for part, _, _ in self.sparse_all_reduce:
            lines.append(f"sparse all-reduce {part.part_name}")
        for e in self.ps_entries.values():
            lines.append(f"ps {e.part.part_name} -> rank {e.owner} gate={e.gate} "
                         f"staleness={e.staleness} proxy={e.local_replication}")
        return "\n".join(lines)
