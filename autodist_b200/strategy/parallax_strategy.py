"""``Parallax`` builder: dense gradients by all-reduce, sparse gradients through load-balanced PS.

Reference: ``autodist/strategy/parallax_strategy.py:24-71``. Group ids count
every variable (sparse ones included); sparse PS variables never get a proxy.

With ``reduction_devices="gpu"`` (the owners are the replica GPUs of one NVSwitch box) a row-sparse table of two or more
dimensions is split along axis 0 into one shard per GPU, shard ``i`` owned by GPU ``i``: the layout the peer-memory
kernels serve (rows gathered from their owners inside the lookup kernel, gradient rows added straight into the owners'
shards), so that no replica holds - or reduces - the whole table. The strategy message needs nothing new for this: a
``partitioner`` string and one ``part_config`` per shard, as PartitionedPS writes them.
"""
from autodist_b200.strategy import _placement as P
from autodist_b200.strategy.all_reduce_strategy import AllReduce
from autodist_b200.strategy.ps_strategy import PSLoadBalancing


class Parallax(PSLoadBalancing, AllReduce):
    def __init__(self, chunk_size=128, local_proxy_variable=False, sync=True, staleness=0,
                 all_reduce_spec="NCCL", compressor="NoneCompressor", reduction_devices="cpu"):
        PSLoadBalancing.__init__(self, local_proxy_variable, sync, staleness, reduction_devices)
        AllReduce.__init__(self, chunk_size, all_reduce_spec, compressor)

    def build(self, graph_item, resource_spec):
        s = self._new_strategy(resource_spec)
        self._begin(resource_spec)
        gpus = P.reduction_devices(resource_spec, "gpu") if self._placement == "gpu" and resource_spec.num_gpus else []
        for idx, var in enumerate(graph_item.trainable_var_op_to_var.values()):
            if var.sparse_grad and len(gpus) > 1 and len(var.shape) >= 2 and int(var.shape[0]) >= len(gpus) and not var.in_control_flow:
                node = self._row_sharded_node(var, gpus)
            elif var.sparse_grad:
                node = self._gen_ps_node_config(var, False, self._sync, self._staleness)
            else:
                node = self._gen_all_reduce_node_config(var.name, group=idx // self.chunk_size)
            s.node_config.append(node)
        return s

    def _row_sharded_node(self, var, gpus):
        node = P.strategy_pb2.Strategy.Node()
        node.var_name = var.name
        node.partitioner = P.partition_string(len(var.shape), 0, len(gpus))
        for i, dev in enumerate(gpus):
            P.fill_ps(node.part_config.add(var_name=P.part_name(var.name, i)), dev, False, self._sync, self._staleness)
            self._greedy.add(dev, P.byte_size_load_fn(var) / len(gpus))
        return node
