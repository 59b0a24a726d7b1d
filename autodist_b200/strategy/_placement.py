"""Shared arithmetic of the strategy builders: shard counts, byte loads, greedy placement."""
import math

from autodist_b200.proto import strategy_pb2, synchronizers_pb2


def byte_size_load_fn(var):
    """Load of a variable = number of elements x element size."""
    return float(var.byte_size)


def min_divisor_shards(n):
    """Smallest divisor >= 2 of ``n``; ``n`` itself when prime (reference
    ``partitioned_ps_strategy.py:126-135``)."""
    for i in range(2, n):
        if n % i == 0:
            return i
    return n


def first_non_divisor_shards(n):
    """Smallest ``i >= 2`` that does not divide ``n`` (``uneven_partition_ps_strategy.py:125-135``)."""
    for i in range(2, n):
        if n % i > 0:
            return i
    return n


def partition_string(ndim, axis, num_shards):
    parts = ["1"] * ndim
    parts[axis] = str(num_shards)
    return ",".join(parts)


def part_name(var_name, index):
    op_name = var_name[:-2] if var_name.endswith(":0") else var_name
    return f"{op_name}/part_{index}:0"


class GreedyLoads:
    """Accumulated byte load per reduction device; ties keep declaration order."""

    def __init__(self, devices):
        self.loads = {d: 0.0 for d in devices}

    def __len__(self):
        return len(self.loads)

    def least_loaded(self, count=1):
        order = sorted(self.loads, key=self.loads.get)
        if count > len(order):
            order = order * math.ceil(count / len(order))  # round-robin in greedy order
        return order[:count]

    def add(self, device, nbytes):
        self.loads[device] += nbytes


def reduction_devices(resource_spec, placement="cpu"):
    """Candidate parameter-server devices.

    ``"cpu"`` is the reference's rule (every CPU device). ``"gpu"`` makes the
    replica GPUs themselves the owners, which is what a single NVSwitch box
    wants: the owner GPU receives the reduce-scatter and runs the update.
    """
    if placement == "gpu" and resource_spec.num_gpus:
        return [k for k, _ in resource_spec.gpu_devices]
    return [k for k, _ in resource_spec.cpu_devices]


def ps_node(var_name, destination, local_replication, sync, staleness):
    node = strategy_pb2.Strategy.Node()
    node.var_name = var_name
    fill_ps(node, destination, local_replication, sync, staleness)
    return node


def fill_ps(node, destination, local_replication, sync, staleness):
    ps = node.PSSynchronizer
    ps.reduction_destination = destination
    ps.local_replication = bool(local_replication)
    ps.sync = bool(sync)
    ps.staleness = int(staleness)


def fill_all_reduce(node, group, spec="NCCL", compressor="NoneCompressor", power_sgd_rank=0):
    ar = node.AllReduceSynchronizer
    ar.spec = synchronizers_pb2.AllReduceSynchronizer.Spec.Value(spec)
    ar.compressor = synchronizers_pb2.AllReduceSynchronizer.Compressor.Value(compressor)
    ar.group = int(group)
    if power_sgd_rank:
        ar.power_sgd_rank = int(power_sgd_rank)


def all_reduce_node(var_name, group, spec="NCCL", compressor="NoneCompressor", power_sgd_rank=0):
    node = strategy_pb2.Strategy.Node()
    node.var_name = var_name
    fill_all_reduce(node, group, spec, compressor, power_sgd_rank)
    return node
