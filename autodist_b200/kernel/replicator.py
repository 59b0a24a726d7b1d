"""Replication pass.

The reference imports the graph once per local GPU under ``AutoDist-Replica-<i>/``
name scopes inside one process (``autodist/kernel/replicator.py:60-171``). Here a
replica *is* a process: the pass works out, from the strategy's replica list and
the rank of this process, which replica this process runs, which ranks share
its node (the "local replicas" that split a fed batch between them) and how
many nodes there are.
"""
from autodist_b200.kernel.kernel import Kernel
from autodist_b200.kernel.plan import ReplicaInfo


def _host_of(resolved):
    # "/job:worker/task:<k>/device:..." -> k
    return resolved.split("/task:")[1].split("/")[0]


class Replicator(Kernel):
    def __init__(self, key, replicas, rank):
        super().__init__(key)
        self._replicas = list(replicas)
        self._rank = rank

    def _apply(self):
        if not 0 <= self._rank < len(self._replicas):
            raise ValueError(f"rank {self._rank} has no replica among {len(self._replicas)} replica devices")
        mine = _host_of(self._replicas[self._rank])
        local = [r for r, dev in enumerate(self._replicas) if _host_of(dev) == mine]
        workers = len({_host_of(d) for d in self._replicas})
        return ReplicaInfo(rank=self._rank, world_size=len(self._replicas), device=self._replicas[self._rank],
                           replicas=self._replicas, local_ranks=local, num_workers=workers)
