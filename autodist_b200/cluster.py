"""Cluster: which processes make up the job and how they find each other.

Capability parity with ``autodist/cluster.py:51-374``. The reference starts one
TensorFlow gRPC server per node and lets one client process per node drive all
of that node's GPUs; here the job is one process per replica device, joined in a
single ``torch.distributed`` world (NCCL between GPUs, gloo between CPU slots).
``start()`` therefore only fixes the rendezvous endpoint; the processes
themselves are started by the ``Coordinator``. Remote nodes are reached with the
system ``ssh`` / ``scp`` binaries using the resource spec's SSH configuration.
"""
import atexit
import json
import os
import shlex
import socket
import subprocess
from abc import ABCMeta, abstractmethod

from autodist_b200 import const
from autodist_b200.const import ENV
from autodist_b200.resource_spec import DeviceSpec
from autodist_b200.utils import logging
from autodist_b200.utils.network import is_local_address


def _free_port(lo, hi):
    for port in range(lo + (os.getpid() % 500), hi):
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", port))
                return port
            except OSError:
                continue
    raise RuntimeError("no free rendezvous port in %d-%d" % (lo, hi))


class Cluster(metaclass=ABCMeta):
    def __init__(self, resource_spec):
        self._resource_spec = resource_spec
        self._chief = resource_spec.chief
        self._nodes = sorted(resource_spec.nodes)
        self._replicas = list(resource_spec.replica_devices)
        self._port = None
        self.subprocesses = []
        self._started = False
        logging.debug("ClusterSpec nodes: %s", self._nodes)

    # -- description -------------------------------------------------------------------
    @property
    def nodes(self):
        return list(self._nodes)

    @property
    def replica_devices(self):
        return list(self._replicas)

    @property
    def world_size(self):
        return len(self._replicas)

    @property
    def cluster_spec(self):
        """``{"worker": ["ip:port", ...]}`` in sorted-node order (task index = position)."""
        port = self._port or const.DEFAULT_PORT_RANGE[0]
        return {"worker": [f"{ip}:{port}" for ip in self._nodes]}

    def is_chief(self, address=None):
        address = address or self.get_local_address()
        return address == self._chief

    def get_address_from_task(self, job_name, task_index):
        return self.cluster_spec[job_name][task_index].rsplit(":", 1)[0]

    def get_local_address(self):
        """This process's node address: ``AUTODIST_WORKER`` names the replica device on workers."""
        worker = ENV.AUTODIST_WORKER.val
        if worker:
            return worker.rsplit(":", 2)[0] if worker.count(":") >= 2 else worker
        return self._chief

    def get_local_worker_task_index(self):
        return self._nodes.index(self.get_local_address())

    def get_local_session_target(self):
        return f"{self.master_address}:{self.master_port}"

    def ranks_of_node(self, address):
        return [r for r, dev in enumerate(self._replicas) if DeviceSpec.from_string(dev).host_address == address]

    @property
    def chief_rank(self):
        return self.ranks_of_node(self._chief)[0]

    def local_rank_of(self, rank):
        """Index of the CUDA device (or CPU slot) that ``rank`` drives on its node."""
        return DeviceSpec.from_string(self._replicas[rank]).device_index

    # -- rendezvous ----------------------------------------------------------------------
    @property
    def master_address(self):
        if len(self._nodes) == 1 or is_local_address(self._chief) and len(self._nodes) == 1:
            return "127.0.0.1"
        return self._chief

    @property
    def master_port(self):
        if self._port is None:
            env_port = os.environ.get("MASTER_PORT")
            self._port = int(env_port) if env_port else _free_port(*const.DEFAULT_PORT_RANGE)
        return self._port

    def start(self):
        """Fix the rendezvous endpoint and export it (chief only; workers inherit it)."""
        if self._started:
            return
        os.environ.setdefault("MASTER_ADDR", self.master_address)
        os.environ["MASTER_PORT"] = str(self.master_port)
        self._started = True
        atexit.register(self.terminate)
        logging.debug("rendezvous at %s:%s", os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"])

    def terminate(self):
        for proc in self.subprocesses:
            if proc.poll() is None:
                try:
                    os.killpg(os.getpgid(proc.pid), 15)
                except (ProcessLookupError, PermissionError):
                    pass
        self.subprocesses = []

    # -- remote execution ---------------------------------------------------------------
    @abstractmethod
    def remote_exec(self, args, hostname):
        """Run ``args`` (list of str) on ``hostname``; returns a ``Popen`` (``None`` on dry run)."""

    @abstractmethod
    def remote_copy(self, local_path, remote_path, hostname):
        """Copy a file to ``hostname``."""

    @abstractmethod
    def remote_file_write(self, remote_path, data, hostname):
        """Write ``data`` (str) to a file on ``hostname``."""


class SSHCluster(Cluster):
    """Cluster whose remote nodes are driven over SSH."""

    def __init__(self, resource_spec):
        super().__init__(resource_spec)
        self._ssh_conf = resource_spec.ssh_config_map

    def _ssh_base(self, hostname, binary="ssh"):
        conf = self._ssh_conf[hostname]
        cmd = [binary, "-o", "StrictHostKeyChecking=no"]
        if conf.key_file:
            cmd += ["-i", conf.key_file]
        cmd += ["-P" if binary == "scp" else "-p", str(conf.port)]
        return cmd, conf

    def remote_command(self, args, hostname, extra_env=None):
        """The full ssh command line (list) that would run ``args`` on ``hostname``."""
        base, conf = self._ssh_base(hostname)
        env = dict(conf.env)
        env.update(extra_env or {})
        pieces = []
        if conf.python_venv:
            pieces.append(conf.python_venv + ";")
        pieces += [f"{k}={shlex.quote(str(v))}" for k, v in env.items()]
        pieces += [shlex.quote(a) for a in args]
        target = f"{conf.username}@{hostname}" if conf.username else hostname
        return base + ["-tt", target, "bash -c " + shlex.quote(" ".join(pieces))]

    def remote_exec(self, args, hostname, extra_env=None):
        cmd = self.remote_command(args, hostname, extra_env)
        if ENV.AUTODIST_DEBUG_REMOTE.val:
            logging.info("[dry run] %s", " ".join(cmd))
            return None
        proc = subprocess.Popen(cmd, start_new_session=True)
        self.subprocesses.append(proc)
        return proc

    def remote_copy(self, local_path, remote_path, hostname):
        base, conf = self._ssh_base(hostname, "scp")
        target = f"{conf.username}@{hostname}" if conf.username else hostname
        cmd = base + [local_path, f"{target}:{remote_path}"]
        if ENV.AUTODIST_DEBUG_REMOTE.val:
            logging.info("[dry run] %s", " ".join(cmd))
            return None
        return subprocess.run(cmd, check=True)

    def remote_file_write(self, remote_path, data, hostname):
        cmd = self.remote_command(["bash", "-c", f"mkdir -p {shlex.quote(os.path.dirname(remote_path))} && "
                                   f"cat > {shlex.quote(remote_path)}"], hostname)
        if ENV.AUTODIST_DEBUG_REMOTE.val:
            logging.info("[dry run] write %d bytes to %s:%s", len(data), hostname, remote_path)
            return None
        return subprocess.run(cmd, input=data.encode(), check=True)

    def dump_cluster_spec(self, path):
        with open(path, "w") as f:
            json.dump(self.cluster_spec, f)
