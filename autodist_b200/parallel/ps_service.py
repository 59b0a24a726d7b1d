"""Relaxed parameter-server modes: bounded staleness (SSP) and fully asynchronous updates.

In the reference these modes are built from shared accumulators and token
queues placed on the parameter-server device
(``autodist/kernel/synchronization/ps_synchronizer.py:335-458,557-633``): with
``staleness > 0`` every worker's gradient is applied on its own as it arrives and
a worker may run at most ``staleness`` steps ahead of the slowest one; with
``sync=False`` there is no gate at all.

Collectives cannot express "apply whatever arrives": they need every rank in
every call. So the relaxed modes use a small host-side service instead. Every
rank that owns parameter-server parts runs a server thread; ranks push their
gradients for those parts to the owner (which applies them immediately under a
lock with the owner's optimizer) and pull the current values back. The lowest
owner rank also keeps the step clocks that implement the staleness gate. The
waits are bounded: a gate that does not open within ``AUTODIST_GATE_TIMEOUT``
seconds raises instead of hanging.
"""
import os
import threading
import time
from multiprocessing.connection import Client, Listener

import torch

from autodist_b200.utils import logging

def _base_port():
    return int(os.environ.get("MASTER_PORT", "29500")) + 101


def _own_host(single_node):
    """Address this rank's listener binds to: loopback when every rank runs on this machine, else this node's own address
    (``AUTODIST_NODE_ADDR``, or what the host name resolves to) - never the chief's address on another node."""
    if single_node:
        return "127.0.0.1"
    addr = os.environ.get("AUTODIST_NODE_ADDR")
    if addr:
        return addr
    import socket
    return socket.gethostbyname(socket.gethostname())


def _job_secrets(engine):
    """(authentication key, host of every rank), agreed over the job's process group.

    The connections carry pickles, so the key must not be guessable: rank 0 draws 32 random bytes per job and the
    process group (already restricted to the job's ranks) hands them to the others. A single process needs none."""
    import torch.distributed as dist
    world = engine.world_size
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    single_node = local_world >= world
    if world <= 1 or not dist.is_initialized():
        return os.urandom(32), {0: "127.0.0.1"}
    group = getattr(engine.backend, "group", None)
    box = [os.urandom(32) if engine.rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    hosts = [None] * world
    dist.all_gather_object(hosts, _own_host(single_node), group=group)
    return box[0], dict(enumerate(hosts))


class StepClocks:
    """Per-rank step counters with the SSP rule ``clock[r] - min(clock) <= staleness``."""

    def __init__(self, ranks):
        self._clock = {r: 0 for r in ranks}
        self._cv = threading.Condition()
        self.max_lead_seen = {r: 0 for r in ranks}

    def advance_and_wait(self, rank, staleness, timeout):
        deadline = time.monotonic() + timeout
        with self._cv:
            self._clock[rank] += 1
            self._cv.notify_all()
            while staleness is not None:
                lead = self._clock[rank] - min(self._clock.values())
                if lead <= staleness:
                    break
                left = deadline - time.monotonic()
                if left <= 0:
                    return False, lead
                self._cv.wait(timeout=min(left, 0.5))
            lead = self._clock[rank] - min(self._clock.values()) if self._clock else 0
            self.max_lead_seen[rank] = max(self.max_lead_seen.get(rank, 0), lead)
            return True, lead

    def leave(self, rank):
        with self._cv:
            self._clock.pop(rank, None)
            self._cv.notify_all()


class PSServer(threading.Thread):
    """Owner-side service: applies pushed gradients, serves pulls, keeps the clocks (lowest owner only)."""

    def __init__(self, engine, owner, ranks, keeps_clocks, host="127.0.0.1", authkey=None):
        super().__init__(daemon=True, name=f"ps-server-{owner}")
        self.engine = engine
        self.owner = owner
        self.lock = threading.Lock()
        self.clocks = StepClocks(ranks) if keeps_clocks else None
        self.listener = Listener((host, _base_port() + owner), authkey=authkey)
        self._stop = False
        self.pushes_applied = 0

    def run(self):
        while not self._stop:
            try:
                conn = self.listener.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn):
        try:
            while True:
                try:
                    msg = conn.recv()
                except (EOFError, OSError):
                    return
                kind = msg[0]
                if kind == "push":
                    _, rank, op_index, grads = msg
                    with self.lock:
                        self.engine._apply_pushed(op_index, grads)
                        self.pushes_applied += 1
                    conn.send(("ok",))
                elif kind == "pull":
                    with self.lock:
                        conn.send(("values", self.engine._owned_values()))
                elif kind == "gate":
                    _, rank, staleness, timeout = msg
                    ok, lead = self.clocks.advance_and_wait(rank, staleness, timeout)
                    conn.send(("gate", ok, lead))
                elif kind == "leave":
                    if self.clocks is not None:
                        self.clocks.leave(msg[1])
                    conn.send(("ok",))
                elif kind == "close":
                    conn.send(("ok",))
                    return
        finally:
            conn.close()

    def stop(self):
        self._stop = True
        try:
            self.listener.close()
        except OSError:
            pass


class RelaxedPSClient:
    """Per-rank driver of the relaxed modes; owns this rank's server if it is an owner."""

    def __init__(self, engine):
        self.engine = engine
        self.plan = engine.plan
        self.rank = engine.rank
        self.owners = sorted(self.plan.ps_by_owner())
        self.staleness = self.plan.staleness if self.plan.gate_mode == "stale" else None
        self.timeout = float(os.environ.get("AUTODIST_GATE_TIMEOUT", "120"))
        self.server = None
        self.last_lead = 0
        self.max_lead = 0
        authkey, hosts = _job_secrets(engine)
        if self.rank in self.owners:
            self.server = PSServer(engine, self.rank, range(engine.world_size), self.rank == self.owners[0],
                                   host=hosts.get(self.rank, "127.0.0.1"), authkey=authkey)
            self.server.start()
        engine.backend.barrier()  # every listener is up before anybody connects
        self.conns = {o: Client((hosts.get(o, "127.0.0.1"), _base_port() + o), authkey=authkey) for o in self.owners}

    def _call(self, owner, msg):
        c = self.conns[owner]
        c.send(msg)
        return c.recv()

    def before_step(self):
        return

    def push_and_pull(self, train_op):
        eng = self.engine
        by_owner = self.plan.ps_by_owner()
        for owner in self.owners:
            grads = {}
            for e in by_owner[owner]:
                p = eng._params[e.part.var_name]
                g = eng._dense_grad(p)
                grads[e.part.part_name] = e.part.view(g).detach().cpu().contiguous().numpy()
            self._call(owner, ("push", self.rank, train_op.optimizer_index, grads))
        for p_name in {e.part.var_name for e in self.plan.ps_entries.values()}:
            eng._params[p_name].grad = None  # applied remotely; the local optimizer must not re-apply
        if self.plan.gate_mode == "stale":
            _, ok, lead = self._call(self.owners[0], ("gate", self.rank, self.staleness, self.timeout))
            if not ok:
                raise TimeoutError(f"rank {self.rank}: staleness gate did not open in {self.timeout}s (lead {lead})")
            self.last_lead = lead
            self.max_lead = max(self.max_lead, lead)
        for owner in self.owners:
            _, values = self._call(owner, ("pull", self.rank))
            for e in by_owner[owner]:
                dst = e.part.view(eng._params[e.part.var_name].data)
                dst.copy_(torch.from_numpy(values[e.part.part_name]).to(dst.device).view(dst.shape))

    def close(self):
        for owner, c in self.conns.items():
            try:
                if owner == self.owners[0]:
                    c.send(("leave", self.rank))
                    c.recv()
                c.send(("close",))
                c.recv()
                c.close()
            except (OSError, EOFError):
                pass
        self.conns = {}
        try:
            self.engine.backend.barrier()
        except Exception:  # a peer may already be gone at shutdown
            pass
        if self.server is not None:
            self.server.stop()
