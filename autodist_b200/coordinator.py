"""Coordinator: the chief starts the other ranks and watches them.

Capability parity with ``autodist/coordinator.py:27-110``: every other replica
re-executes the user's script with ``AUTODIST_WORKER`` / ``AUTODIST_STRATEGY_ID``
set (remote ones after the strategy file has been copied over), and a watcher
thread per worker reacts to a non-zero exit. The reference ``os._exit(1)``s the
chief; here the failure is recorded, the remaining workers are torn down and the
next ``session.run`` raises ``WorkerFailure`` in the chief.
"""
import os
import subprocess
import sys
import threading

from autodist_b200.const import ENV
from autodist_b200.utils import logging
from autodist_b200.utils.network import is_local_address


class WorkerFailure(RuntimeError):
    pass


class Coordinator:
    def __init__(self, strategy, cluster):
        self._strategy = strategy
        self.cluster = cluster
        self.threads = []
        self.procs = {}
        self.failure = None
        self._lock = threading.Lock()

    def _worker_env(self, rank):
        device = self.cluster.replica_devices[rank]
        env = {
            ENV.AUTODIST_WORKER.name: device,
            ENV.AUTODIST_STRATEGY_ID.name: self._strategy.id,
            ENV.AUTODIST_RANK.name: str(rank),
            "RANK": str(rank),
            "WORLD_SIZE": str(self.cluster.world_size),
            "LOCAL_RANK": str(self.cluster.local_rank_of(rank)),
            "MASTER_ADDR": os.environ.get("MASTER_ADDR", self.cluster.master_address),
            "MASTER_PORT": str(self.cluster.master_port),
        }
        for flag in (ENV.AUTODIST_MIN_LOG_LEVEL, ENV.AUTODIST_IS_TESTING, ENV.AUTODIST_PATCH_TF,
                     ENV.AUTODIST_INTERNAL_TF, ENV.SYS_DATA_PATH, ENV.SYS_RESOURCE_PATH,
                     ENV.AUTODIST_FETCH_MODE, ENV.AUTODIST_COMM):
            if os.environ.get(flag.name) is not None:
                env[flag.name] = os.environ[flag.name]
        # every other AUTODIST_* knob the user set (kernel time-outs, flight size, metrics file, step deadline ...) applies
        # to the whole job, so it travels too; the per-rank identity variables above are never overwritten
        for name, value in os.environ.items():
            if name.startswith("AUTODIST_") and name not in env:
                env[name] = value
        return env

    def launch_clients(self):
        """Start one process per replica other than the chief's own."""
        argv = [sys.executable, os.path.abspath(sys.argv[0])] + sys.argv[1:]
        chief_rank = self.cluster.chief_rank
        for rank, device in enumerate(self.cluster.replica_devices):
            if rank == chief_rank:
                continue
            host = device.rsplit(":", 2)[0]
            env = self._worker_env(rank)
            if is_local_address(host) or len(self.cluster.nodes) == 1:
                proc = subprocess.Popen(argv, env={**os.environ, **env}, start_new_session=True)
                self.cluster.subprocesses.append(proc)
            else:
                if self._strategy.path:
                    self.cluster.remote_copy(self._strategy.path, self._strategy.path, host)
                proc = self.cluster.remote_exec(argv, host, extra_env=env)
            if proc is None:
                continue  # dry run
            self.procs[rank] = proc
            t = threading.Thread(target=self._watch, args=(rank, proc), daemon=True)
            t.start()
            self.threads.append(t)
        return self.procs

    def _watch(self, rank, proc):
        code = proc.wait()
        if code == 0:
            return
        with self._lock:
            if self.failure is None:
                self.failure = (rank, code)
                logging.error("worker rank %d exited with code %s; stopping the job", rank, code)
        for other_rank, other in self.procs.items():
            if other is not proc and other.poll() is None:
                try:
                    os.killpg(os.getpgid(other.pid), 15)
                except (ProcessLookupError, PermissionError):
                    pass

    def check(self):
        """Raise in the chief if a worker has failed."""
        if self.failure is not None:
            rank, code = self.failure
            raise WorkerFailure(f"worker rank {rank} exited with code {code}")

    def join(self, timeout=None):
        for t in self.threads:
            t.join(timeout)
        self.check()
