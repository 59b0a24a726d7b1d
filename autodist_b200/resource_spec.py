"""Cluster resource description parsed from ``resource_spec.yml``.

Same YAML schema and device-name strings as the reference
(``autodist/resource_spec.py:27-331``): ``nodes: [{address, gpus, cpus, chief,
ssh_config, network_bandwidth}]`` and an optional ``ssh:`` section of named
configurations. Device names are ``"<address>:<CPU|GPU>:<index>"``.

What differs underneath: a node's devices become ranks of one
``torch.distributed`` job (one process per GPU, or per CPU slot on GPU-less
nodes) instead of TensorFlow devices behind a gRPC server, and the default
``network_bandwidth`` of a single-node GPU spec is the NVLink 5 per-direction
figure rather than 1 GbE (multi-node specs keep the reference's default of 1).
"""
import enum
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import yaml

from autodist_b200.utils import logging
from autodist_b200.utils.network import is_local_address, is_loopback_address

NVLINK5_GBPS_PER_DIRECTION = 900 * 8  # 900 GB/s expressed in Gbit/s like the YAML field


class DeviceType(enum.Enum):
    CPU = 0
    GPU = 1


class Connectivity(enum.Enum):
    """How two devices reach each other, ordered from slowest to fastest."""
    ETHERNET = 0
    CPU_TO_GPU = 1
    SAME_GPU = 2
    NVSWITCH = 3


class DeviceSpec:
    """One addressable device: ``host:TYPE:index``."""

    __slots__ = ("host_address", "host_device", "device_type", "device_index")

    def __init__(self, host_address, host_device=None, device_type=DeviceType.CPU, device_index=0):
        self.host_address = host_address
        self.device_type = device_type
        self.device_index = int(device_index)
        # A CPU:0 device is its own host device.
        self.host_device = host_device if host_device is not None else self

    def name_string(self):
        return f"{self.host_address}:{self.device_type.name}:{self.device_index}"

    @classmethod
    def from_string(cls, name):
        host, kind, index = name.rsplit(":", 2)
        host_cpu = cls(host)
        kind = DeviceType[kind.upper()]
        if kind is DeviceType.CPU and int(index) == 0:
            return host_cpu
        return cls(host, host_cpu, kind, int(index))

    def connectivity_with(self, other):
        if self.host_address != other.host_address:
            return Connectivity.ETHERNET
        if self.device_type is DeviceType.GPU and other.device_type is DeviceType.GPU:
            return Connectivity.SAME_GPU if self.device_index == other.device_index else Connectivity.NVSWITCH
        return Connectivity.CPU_TO_GPU

    def __eq__(self, other):
        return isinstance(other, DeviceSpec) and self.name_string() == other.name_string()

    def __hash__(self):
        return hash(self.name_string())

    def __repr__(self):
        return f"<DeviceSpec: {self.name_string()}>"

    __str__ = name_string


@dataclass
class SSHConfig:
    """Launch configuration for one group of remote nodes (``ssh:`` section entry)."""
    username: str = ""
    port: int = 22
    python_venv: str = ""
    key_file: Optional[str] = None
    env: Dict[str, str] = field(default_factory=dict)

    @classmethod
    def from_info(cls, info):
        env = {"AUTODIST_MIN_LOG_LEVEL": os.environ.get("AUTODIST_MIN_LOG_LEVEL", "INFO")}
        env.update({str(k): str(v) for k, v in (info.get("shared_envs") or {}).items()})
        return cls(username=info.get("username", ""), port=int(info.get("port", 22)),
                   python_venv=info.get("python_venv", ""), key_file=info.get("key_file"), env=env)

    @property
    def pkey(self):
        """Load the private key lazily (paramiko is only needed for real multi-node launches)."""
        if not self.key_file:
            return None
        import paramiko
        return paramiko.RSAKey.from_private_key_file(os.path.expanduser(os.path.abspath(self.key_file)))


class SSHConfigMap(dict):
    """``hostname -> SSHConfig`` built from the ``ssh:`` section and each node's ``ssh_config``."""

    def __init__(self, info, node_groups, node_gpu_devices):
        super().__init__()
        confs = {name: SSHConfig.from_info(cfg) for name, cfg in (info or {}).items()}
        for hostname, group in node_groups.items():
            if group is None:
                continue
            if group not in confs:
                raise ValueError(f"ssh_config '{group}' of node {hostname} is not defined in the ssh section")
            conf = SSHConfig(**{**confs[group].__dict__, "env": dict(confs[group].env)})
            if hostname not in node_gpu_devices:
                # GPU-less node: hide accelerators from whatever is launched there.
                conf.env["CUDA_VISIBLE_DEVICES"] = ""
            self[hostname] = conf


class ResourceSpec:
    """Devices, chief, SSH groups and bandwidths of the cluster."""

    def __init__(self, resource_file=None, resource_info=None):
        self._devices: Dict[str, DeviceSpec] = {}
        self._chief = None
        self._ssh_group: Dict[str, Optional[str]] = {}
        self._ssh_config_map = {}
        self._bandwidth: Dict[str, float] = {}
        if resource_file is not None:
            with open(resource_file, "r") as f:
                resource_info = yaml.safe_load(f)
        if resource_info is not None:
            self._load(dict(resource_info))

    # ---- construction -------------------------------------------------
    @classmethod
    def local(cls, num_gpus=0, num_cpus=1, address="localhost"):
        """A single-node spec without a file: ``num_gpus`` GPUs, or ``num_cpus`` CPU slots."""
        node = {"address": address, "chief": True}
        if num_gpus:
            node["gpus"] = list(range(num_gpus))
        else:
            node["cpus"] = list(range(num_cpus))
        return cls(resource_info={"nodes": [node]})

    def _load(self, info):
        nodes = info.pop("nodes", None) or []
        for node in nodes:
            self._add_node(node, len(nodes))
        if self._chief is None:
            raise ValueError('Must provide "chief: true" in one of the nodes in resource spec.')
        if is_local_address(self._chief):
            self._ssh_config_map = SSHConfigMap(info.pop("ssh", {}), self._ssh_group, self.node_gpu_devices)

    def _add(self, dev):
        self._devices.setdefault(dev.name_string(), dev)

    def _add_node(self, node, num_nodes):
        host = str(node["address"])
        if num_nodes > 1 and is_loopback_address(host):
            raise ValueError("Can't (currently) use a loopback address when there are multiple nodes.")
        if node.get("chief") or num_nodes == 1:
            logging.debug("Chief: %s", host)
            self._chief = host
        host_cpu = DeviceSpec(host)
        self._add(host_cpu)
        gpus = sorted(set(node.get("gpus") or []))
        if not gpus:
            for idx in sorted(set(node.get("cpus") or []) - {0}):
                self._add(DeviceSpec(host, host_cpu, DeviceType.CPU, idx))
        for idx in gpus:
            self._add(DeviceSpec(host, host_cpu, DeviceType.GPU, idx))
        self._ssh_group[host] = node.get("ssh_config")
        if self._ssh_group[host] is None and self._chief != host:
            raise ValueError("Need to define SSH groups for all non-chief nodes.")
        if node.get("network_bandwidth"):
            self._bandwidth[host] = node["network_bandwidth"]
        else:
            self._bandwidth[host] = 1

    # ---- queries --------------------------------------------------------
    @property
    def chief(self):
        return self._chief

    @property
    def devices(self):
        return self._devices.items()

    @property
    def nodes(self):
        return {d.host_address for d in self._devices.values()}

    def _of_type(self, kind):
        return {k: v for k, v in self._devices.items() if v.device_type is kind}

    @property
    def cpu_devices(self):
        return self._of_type(DeviceType.CPU).items()

    @property
    def gpu_devices(self):
        return self._of_type(DeviceType.GPU).items()

    @property
    def num_cpus(self):
        return len(self._of_type(DeviceType.CPU))

    @property
    def num_gpus(self):
        return len(self._of_type(DeviceType.GPU))

    @staticmethod
    def _by_node(items):
        out: Dict[str, List[str]] = {}
        for name, dev in items:
            out.setdefault(dev.host_address, []).append(name)
        return out

    @property
    def node_gpu_devices(self):
        return self._by_node(self.gpu_devices)

    @property
    def node_cpu_devices(self):
        return self._by_node(self.cpu_devices)

    @property
    def ssh_config_map(self):
        return self._ssh_config_map

    @property
    def ssh_group(self):
        return self._ssh_group

    @property
    def network_bandwidth(self):
        return self._bandwidth

    # ---- additions used by the rank launcher and the cost model ----------
    @property
    def replica_devices(self):
        """Replica list rule shared by all builders: every GPU, plus the CPUs of GPU-less nodes.

        Ordered by sorted node address then device index, which is also the
        global rank order of the job (reference: ``ps_strategy.py:42-45`` for the
        rule, ``cluster.py:78-80`` for the sorted-node task order).
        """
        gpu_nodes = self.node_gpu_devices
        out = []
        for host in sorted(self.nodes):
            if host in gpu_nodes:
                out += sorted(gpu_nodes[host], key=lambda n: int(n.rsplit(":", 1)[1]))
            else:
                out += sorted(self.node_cpu_devices.get(host, []), key=lambda n: int(n.rsplit(":", 1)[1]))
        return out

    def link_bandwidth_gbps(self, a: DeviceSpec, b: DeviceSpec):
        """Gbit/s between two devices for the cost model."""
        kind = a.connectivity_with(b)
        if kind is Connectivity.NVSWITCH:
            return NVLINK5_GBPS_PER_DIRECTION
        if kind is Connectivity.SAME_GPU:
            return 8 * 6500  # HBM copy
        if kind is Connectivity.CPU_TO_GPU:
            return 8 * 55    # PCIe gen5 x16, one direction
        return min(self._bandwidth.get(a.host_address, 1), self._bandwidth.get(b.host_address, 1))
