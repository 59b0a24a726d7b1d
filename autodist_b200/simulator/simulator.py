"""Predicts the per-step synchronisation time of a strategy and ranks strategies.

The prediction walks the strategy's nodes the way the transformer would: all-reduce nodes are grouped into buckets
(one collective per group, compressed wire width where a compressor narrows it), parameter-server nodes become a
reduce to the owner + the owner's update + a publish (or, when shards are spread over all GPUs, a reduce-scatter and
an all-gather), sparse nodes move only the rows touched. Dataset records follow the layout the reference documents
(``autodist/simulator/dataset/README.md:9-65``): resource spec, runtime ``{runtime: [...], average: x}``, strategy.
"""
import os
from collections import defaultdict

import yaml

from autodist_b200.proto import synchronizers_pb2
from autodist_b200.simulator.cost_model import NVSwitchCostModel

_WIRE_FACTOR = {"NoneCompressor": 1.0, "HorovodCompressor": 0.5, "HorovodCompressorEF": 0.5}
# HBM bytes moved by pack + unpack per byte of fp32 gradient
_PACK_TRAFFIC = {"HorovodCompressor": 1.0 + 0.5 + 0.5 + 1.0, "HorovodCompressorEF": 1.0 + 2.0 + 0.5 + 0.5 + 1.0}


class Simulator:
    def __init__(self, resource_spec, cost_model=None, sparse_rows_per_step=4096, overlap=0.7):
        self.resource_spec = resource_spec
        n = max(1, len(resource_spec.replica_devices))
        nodes = max(1, len(resource_spec.nodes))
        bw = min(resource_spec.network_bandwidth.values()) if resource_spec.network_bandwidth else None
        self.model = cost_model or NVSwitchCostModel(n // nodes if nodes > 1 else n, num_nodes=nodes, ethernet_gbps=bw)
        self.world = n
        self.sparse_rows = sparse_rows_per_step
        self.overlap = overlap          # fraction of communication hidden behind the backward pass

    def _var(self, graph_item, name):
        return graph_item.variables[name]

    def simulate(self, strategy, graph_item, compute_ms=0.0):
        """Predicted step time in milliseconds (``compute_ms`` + exposed synchronisation + optimizer)."""
        b = self.breakdown(strategy, graph_item)
        return compute_ms + b["exposed_sync_ms"] + b["optimizer_ms"]

    def breakdown(self, strategy, graph_item):
        """``{"sync_ms", "exposed_sync_ms", "optimizer_ms"}`` of one step under ``strategy``."""
        m = self.model
        groups = defaultdict(float)
        sync = 0.0
        opt = 0.0
        owners = defaultdict(float)
        for node in strategy.node_config:
            var = self._var(graph_item, node.var_name)
            parts = list(node.part_config) if node.partitioner and node.part_config else [node]
            share = var.byte_size / len(parts)
            for part in parts:
                which = part.WhichOneof("synchronizer")
                if which == "AllReduceSynchronizer":
                    cfg = part.AllReduceSynchronizer
                    comp = synchronizers_pb2.AllReduceSynchronizer.Compressor.Name(cfg.compressor)
                    if var.sparse_grad:
                        sync += m.sparse_rows(self.sparse_rows * self.world, share / max(var.shape[0], 1) * len(parts))
                    elif comp == "PowerSGDCompressor" and len(var.shape) >= 2:
                        r = max(1, cfg.power_sgd_rank)
                        cols = var.numel // var.shape[0]
                        groups[(cfg.group, comp)] += (var.shape[0] + cols) * r * 4.0 / len(parts)
                    else:
                        groups[(cfg.group, comp)] += share * _WIRE_FACTOR.get(comp, 1.0)
                        # narrowing is an extra pass over HBM on each side of the collective: read the gradient, (read
                        # and write the error-feedback residual,) write the wire copy; read it back and widen it
                        if comp in _PACK_TRAFFIC:
                            sync += share * _PACK_TRAFFIC[comp] / (m.hbm_gbs * 1e9)
                    opt += m.optimizer(var.numel / len(parts))
                elif which == "PSSynchronizer":
                    cfg = part.PSSynchronizer
                    if var.sparse_grad:
                        sync += 2 * m.sparse_rows(self.sparse_rows * self.world, share / max(var.shape[0], 1) * len(parts))
                    else:
                        owners[cfg.reduction_destination] += share
                    opt += m.optimizer(var.numel / len(parts), sharded=False) / max(1, len(parts))
        for nbytes in groups.values():
            sync += m.all_reduce(nbytes)
        if owners:
            spread = len(owners) >= self.world and self.world > 1
            total = sum(owners.values())
            if spread:
                sync += m.reduce_scatter(total) + m.all_gather(total / 2.0)      # bf16 parameters come back
            else:
                worst = max(owners.values())
                sync += m.reduce_to_owner(worst) + m.broadcast_from_owner(worst / 2.0)
        exposed = sync * (1.0 - self.overlap)
        return {"sync_ms": sync * 1e3, "exposed_sync_ms": exposed * 1e3, "optimizer_ms": opt * 1e3}

    # ---- dataset records -----------------------------------------------------------------------------
    @staticmethod
    def record(directory, resource_file, strategy, runtimes_s):
        os.makedirs(directory, exist_ok=True)
        path = strategy.serialize(os.path.join(directory, f"strategy_{strategy.id}"))
        with open(os.path.join(directory, f"runtime_{strategy.id}.yml"), "w") as f:
            yaml.safe_dump({"runtime": [float(x) for x in runtimes_s],
                            "average": float(sum(runtimes_s) / max(1, len(runtimes_s))),
                            "resource_spec": resource_file, "strategy": os.path.basename(path)}, f)
        return path

    @staticmethod
    def load_records(directory):
        out = []
        for name in sorted(os.listdir(directory)):
            if name.startswith("runtime_") and name.endswith(".yml"):
                with open(os.path.join(directory, name)) as f:
                    out.append(yaml.safe_load(f))
        return out


def rank_strategies(builders, graph_item, resource_spec, compute_ms=0.0, simulator=None):
    """``[(predicted ms, name, strategy)]`` sorted fastest first. ``builders`` maps names to StrategyBuilder objects."""
    sim = simulator or Simulator(resource_spec)
    ranked = []
    for name, builder in builders.items():
        s = builder.build(graph_item, resource_spec)
        ranked.append((sim.simulate(s, graph_item, compute_ms), name, s))
    ranked.sort(key=lambda t: t[0])
    return ranked
