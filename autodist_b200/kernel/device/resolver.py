"""Device-string resolution: ``"ip:GPU:3"`` -> the rank that drives that device.

The reference maps to TensorFlow device strings ``/job:worker/task:<k>/device:GPU:<i>``
with ``k`` the position of the address among the sorted nodes
(``autodist/kernel/device/resolver.py:25-67``). With one process per device the
resolved form is ``/job:worker/task:<k>/device:<TYPE>:<i>/rank:<r>``; ``rank_of``
extracts ``r``. A CPU parameter-server destination on a node resolves to the rank
of that node's first replica (the process that hosts the node's CPU-side state).
"""
import re

from autodist_b200.resource_spec import DeviceSpec

_RANK_RE = re.compile(r"/rank:(\d+)$")


class DeviceResolver:
    def __init__(self, cluster):
        self._cluster = cluster
        self._node_order = sorted(cluster.nodes)
        self._replicas = list(cluster.replica_devices)

    def _rank_for(self, spec: DeviceSpec):
        name = spec.name_string()
        if name in self._replicas:
            return self._replicas.index(name)
        # Not a replica device (e.g. host CPU of a GPU node): first replica living on that host.
        for r, rep in enumerate(self._replicas):
            if rep.rsplit(":", 2)[0] == spec.host_address:
                return r
        raise ValueError(f"no replica runs on the host of {name}")

    def resolve_to_device_str(self, device):
        if isinstance(device, (list, tuple)):
            return [self.resolve_to_device_str(d) for d in device]
        if device.startswith("/job:"):
            return device
        spec = DeviceSpec.from_string(device)
        task = self._node_order.index(spec.host_address)
        return (f"/job:worker/task:{task}/device:{spec.device_type.name}:{spec.device_index}"
                f"/rank:{self._rank_for(spec)}")

    @staticmethod
    def rank_of(resolved):
        m = _RANK_RE.search(resolved)
        if not m:
            raise ValueError(f"{resolved!r} is not a resolved device string")
        return int(m.group(1))
