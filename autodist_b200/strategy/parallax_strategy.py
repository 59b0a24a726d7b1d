"""``Parallax`` builder: dense gradients by all-reduce, sparse gradients through load-balanced PS.

Reference: ``autodist/strategy/parallax_strategy.py:24-71``. Group ids count
every variable (sparse ones included); sparse PS variables never get a proxy.
"""
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
        for idx, var in enumerate(graph_item.trainable_var_op_to_var.values()):
            if var.sparse_grad:
                node = self._gen_ps_node_config(var, False, self._sync, self._staleness)
            else:
                node = self._gen_all_reduce_node_config(var.name, group=idx // self.chunk_size)
            s.node_config.append(node)
        return s
