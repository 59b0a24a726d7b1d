"""Step engine: executes a ``DistributedPlan`` around the captured forward / backward.

This is the part of the reference that lives inside the transformed TensorFlow
graph (``autodist/kernel/synchronization/*``: aggregate, apply on the owner,
refresh readers). One engine runs per rank. Per training step:

1. forward of the requested fetches (+ the loss) through a compiled fx module,
2. ``loss.backward()``,
3. every all-reduce bucket: pack member gradients, compressor + mean all-reduce,
   unpack; row-sparse members: exchange (indices, values) and average,
4. every parameter-server part: mean-reduce to its owner rank,
5. the local optimizer (re-created from the captured class / arguments over the
   parameters and shard views this rank updates) takes its step,
6. owners publish updated shards to the other ranks (at once when the strategy
   asked for a local mirror, else lazily before the next read).

The engine is device-agnostic torch code on top of a communication backend; the
fused sm_100a path (``fused_engine.py``) overrides steps 3-6 with kernels that
do the reduction, the update and the re-distribution over NVSwitch peer memory.
"""
from typing import Dict, List, Optional

import warnings

import torch
from torch import nn

from autodist_b200.kernel.common import op_info
from autodist_b200.kernel.synchronization.compressor import Compressor
from autodist_b200.utils import logging

warnings.filterwarnings("ignore", message="Sparse invariant checks")


class _Target:
    """A tensor the local optimizer updates: a full variable or a shard view of it."""

    def __init__(self, var_name, part, full_param, param):
        self.var_name = var_name
        self.part = part            # VarPart or None (whole variable, all parts all-reduced)
        self.full_param = full_param
        self.param = param          # nn.Parameter handed to the optimizer (may be full_param itself)

    def grad_view(self, full_grad):
        return full_grad if self.part is None else self.part.view(full_grad)


class StepEngine:
    def __init__(self, graph_item, plan, backend, device):
        self.item = graph_item
        self.plan = plan
        self.backend = backend
        self.device = torch.device(device)
        self.rank = plan.replica.rank
        self.world_size = plan.replica.world_size
        self.global_step = 0
        self._compiled = {}
        self._flat_buffers: Dict[object, torch.Tensor] = {}
        self._pending_pull = False
        self._params = {name: p for name, p in graph_item.named_parameters()}
        self._move_to_device()
        self._share_initial_values()
        self._compressors = {b.key: self._make_compressor(b) for b in plan.ordered_buckets()}
        self._targets: List[_Target] = []
        self._local_optimizers = []
        from autodist_b200.graph_item import suspend_capture
        with suspend_capture():
            self._build_local_optimizers()
        self._async = None
        if plan.gate_mode != "sync" and self.world_size > 1:
            from autodist_b200.parallel.ps_service import RelaxedPSClient
            self._async = RelaxedPSClient(self)

    # ------------------------------------------------------------------ setup
    def _move_to_device(self):
        if self.device.type == "cpu":
            return
        with torch.no_grad():
            for p in self.item.root.parameters():
                p.data = p.data.to(self.device)
            for name, b in list(self.item.root.named_buffers()):
                b.data = b.data.to(self.device)

    def _share_initial_values(self):
        """Every replica starts from rank 0's initial values (``all_reduce_synchronizer.py:175-196``)."""
        if self.world_size <= 1:
            return
        tensors = [p.data for p in self.item.root.parameters()] + [b.data for b in self.item.root.buffers()]
        by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
        for t in tensors:
            by_dtype.setdefault(t.dtype, []).append(t)
        for dtype, group in by_dtype.items():
            flat = torch.cat([t.reshape(-1) for t in group]) if group else None
            if flat is None or flat.numel() == 0:
                continue
            self.backend.broadcast_(flat, 0)
            off = 0
            for t in group:
                t.copy_(flat[off:off + t.numel()].view_as(t))
                off += t.numel()

    def _make_compressor(self, bucket):
        if bucket.compressor_type == "PowerSGDCompressor":
            return Compressor.create("PowerSGDCompressor", bucket, rank=bucket.power_sgd_rank)
        return Compressor.create(bucket.compressor_type, bucket)

    def _parts_by_var(self):
        """var name -> list of (kind, part, owner) in strategy order."""
        out: Dict[str, list] = {}
        for b in self.plan.ordered_buckets():
            for part in b.parts:
                out.setdefault(part.var_name, []).append(("ar", part, None))
        for part, _, _ in self.plan.sparse_all_reduce:
            out.setdefault(part.var_name, []).append(("ar", part, None))
        for e in self.plan.ps_entries.values():
            out.setdefault(e.part.var_name, []).append(("ps", e.part, e.owner))
        return out

    def _build_local_optimizers(self):
        by_var = self._parts_by_var()
        self._targets_of_param: Dict[int, List[_Target]] = {}
        relaxed = self.plan.gate_mode != "sync" and self.world_size > 1
        self._ps_local = {}
        for oi, info in enumerate(self.item.optimizers):
            groups, group_map = [], []
            ps_groups, ps_map, ps_targets = [], [], []
            for gi, g in enumerate(info.optimizer.param_groups):
                members, ps_members = [], []
                for p in g["params"]:
                    vname = self.item.name_of_parameter(p)
                    entries = by_var.get(vname)
                    if self.world_size <= 1 and entries is None and vname in self.item.updated_variable_names():
                        entries = []
                    if entries is None:
                        continue  # pruned: no gradient reaches this variable
                    if not entries or all(kind == "ar" for kind, _, _ in entries):
                        t = _Target(vname, None, p, p)
                        self._targets.append(t)
                        self._targets_of_param.setdefault(id(p), []).append(t)
                        members.append(p)
                        continue
                    for kind, part, owner in entries:
                        if kind == "ps" and owner != self.rank:
                            continue
                        if part.part_index is None:
                            tp = p
                        else:
                            tp = nn.Parameter(part.view(p.data), requires_grad=True)
                        t = _Target(vname, part, p, tp)
                        if relaxed and kind == "ps":
                            ps_targets.append(t)
                            ps_members.append(tp)
                            continue
                        self._targets.append(t)
                        self._targets_of_param.setdefault(id(p), []).append(t)
                        members.append(tp)
                hyper = {k: v for k, v in g.items() if k != "params"}
                if members:
                    groups.append({**hyper, "params": members})
                    group_map.append(gi)
                if ps_members:
                    ps_groups.append({**hyper, "params": ps_members})
                    ps_map.append(gi)
            if ps_groups:
                self._ps_local[oi] = (info, info.cls(ps_groups, **dict(info.kwargs)), ps_map, ps_targets)
            if groups:
                local = info.cls(groups, **{k: v for k, v in info.kwargs.items()})
                self._local_optimizers.append((info, local, group_map))
            else:
                self._local_optimizers.append((info, None, []))

    # ------------------------------------------------------------------ forward
    def _module_for(self, nodes):
        key = tuple(nodes)
        if key not in self._compiled:
            self._compiled[key] = self.item.compile_fetches(nodes)
        return self._compiled[key]

    def forward(self, nodes, feeds, grad):
        gm, names = self._module_for(tuple(nodes))
        missing = [n for n in names if n not in feeds]
        if missing:
            raise ValueError(f"feed_dict is missing placeholders {missing}")
        args = [feeds[n] for n in names]
        if grad:
            return gm(*args)
        with torch.no_grad():
            return gm(*args)

    # ------------------------------------------------------------------ training step
    def before_read(self):
        """Make lazily refreshed parameter-server variables current."""
        if self._pending_pull:
            self._publish_ps()
            self._pending_pull = False

    def train_step(self, train_op, nodes, feeds):
        self.before_read()
        if self._async is not None:
            self._async.before_step()
        all_nodes = list(nodes)
        if train_op.loss_node not in all_nodes:
            all_nodes.append(train_op.loss_node)
        for p in self._params.values():
            p.grad = None
        values = self.forward(all_nodes, feeds, grad=True)
        loss = values[all_nodes.index(train_op.loss_node)]
        self.backward(loss)
        self.sync_and_update(train_op)
        self.global_step += 1
        return [v.detach() if isinstance(v, torch.Tensor) else v for v in values[:len(nodes)]]

    def train_step_multi(self, train_ops, nodes, feeds):
        """Several train ops fetched by one ``run`` - one per optimizer, over disjoint sets of variables (two networks trained
        against each other, a head with its own optimizer, ...). As in the reference's session, every gradient is taken at
        the values the variables had before the call: one forward pass, each loss differentiated with respect to its own
        optimizer's variables only, one round of gradient synchronisation, then every optimizer steps."""
        if self._async is not None:
            raise NotImplementedError("several train ops in one run() call under a bounded-staleness / asynchronous strategy")
        if len({op.optimizer_index for op in train_ops}) != len(train_ops):
            raise NotImplementedError("several train ops of one optimizer in one run() call")
        owned, seen = [], set()
        for op in train_ops:
            info = self._local_optimizers[op.optimizer_index][0]
            params = op.var_list if op.var_list is not None else [p for g in info.optimizer.param_groups for p in g["params"]]
            if seen & {id(p) for p in params}:
                raise NotImplementedError("train ops fetched together must update disjoint sets of variables")
            seen |= {id(p) for p in params}
            owned.append(list(params))
        self.before_read()
        all_nodes = list(nodes)
        for op in train_ops:
            if op.loss_node not in all_nodes:
                all_nodes.append(op.loss_node)
        for p in self._params.values():
            p.grad = None
        values = self.forward(all_nodes, feeds, grad=True)
        for i, (op, params) in enumerate(zip(train_ops, owned)):
            values[all_nodes.index(op.loss_node)].backward(inputs=params, retain_graph=i + 1 < len(train_ops))
        if self.world_size > 1:
            self._all_reduce_dense()
            self._all_reduce_sparse()
            self._reduce_ps_dense()
            self._reduce_ps_sparse()
        for op in train_ops:
            self._clip(op)
            self._apply_local(op)
        if self.world_size > 1 and self.plan.ps_entries:
            if all(e.local_replication for e in self.plan.ps_entries.values()):
                self._publish_ps()
            else:
                self._pending_pull = True
        self.global_step += 1
        return [v.detach() if isinstance(v, torch.Tensor) else v for v in values[:len(nodes)]]

    def backward(self, loss):
        loss.backward()

    def sync_and_update(self, train_op):
        if self.world_size > 1:
            self._all_reduce_dense()
            self._all_reduce_sparse()
            if self._async is not None:
                self._async.push_and_pull(train_op)
            else:
                self._reduce_ps_dense()
                self._reduce_ps_sparse()
        self._clip(train_op)
        self._apply_local(train_op)
        if self.world_size > 1 and self._async is None and self.plan.ps_entries:
            if all(e.local_replication for e in self.plan.ps_entries.values()):
                self._publish_ps()
            else:
                self._pending_pull = True

    # -- step 3: all-reduce buckets --------------------------------------------------
    def _buffer(self, key, numel, dtype):
        buf = self._flat_buffers.get(key)
        if buf is None or buf.numel() != numel or buf.dtype != dtype:
            buf = torch.zeros(numel, dtype=dtype, device=self.device)
            self._flat_buffers[key] = buf
        return buf

    def _dense_grad(self, p):
        if p.grad is None:
            p.grad = torch.zeros_like(p.data)
        elif p.grad.is_sparse:
            p.grad = p.grad.to_dense()
        return p.grad

    def _all_reduce_dense(self):
        for b in self.plan.ordered_buckets():
            dtype = self._params[b.parts[0].var_name].dtype
            flat = self._buffer(("ar",) + b.key, b.numel, dtype)
            off = 0
            for part, shape in zip(b.parts, b.shapes):
                g = self._dense_grad(self._params[part.var_name])
                flat[off:off + part.numel].view(shape).copy_(part.view(g))
                off += part.numel
            self._compressors[b.key].reduce(flat, self.backend)
            off = 0
            for part, shape in zip(b.parts, b.shapes):
                part.view(self._params[part.var_name].grad).copy_(flat[off:off + part.numel].view(shape))
                off += part.numel

    @staticmethod
    def _rows_of(p):
        """(indices, values) of a row-sparse gradient; a dense one is read as all rows."""
        g = p.grad
        if g is None:
            return (torch.zeros(0, dtype=torch.int64, device=p.device),
                    torch.zeros((0,) + tuple(p.shape[1:]), dtype=p.dtype, device=p.device))
        if g.is_sparse:
            g = g.coalesce()
            return g.indices()[0], g.values()
        return torch.arange(p.shape[0], device=p.device), g

    def _all_reduce_sparse(self):
        done = set()
        for part, _, _ in self.plan.sparse_all_reduce:
            if part.var_name in done:
                continue  # shards of one variable travel together
            done.add(part.var_name)
            p = self._params[part.var_name]
            idx, val = self._rows_of(p)
            gi, gv = self.backend.all_gather_rows(idx, val)
            gv = gv / self.world_size
            p.grad = torch.sparse_coo_tensor(gi.unsqueeze(0), gv, p.shape).coalesce()

    # -- step 4: parameter-server parts --------------------------------------------
    def _reduce_ps_dense(self):
        for owner, entries in sorted(self.plan.ps_by_owner().items()):
            dense = [e for e in entries if not e.part.sparse]
            if not dense:
                continue
            numel = sum(e.part.numel for e in dense)
            dtype = self._params[dense[0].part.var_name].dtype
            flat = self._buffer(("ps", owner), numel, dtype)
            off = 0
            for e in dense:
                g = self._dense_grad(self._params[e.part.var_name])
                shape = e.part.view(g).shape
                flat[off:off + e.part.numel].view(shape).copy_(e.part.view(g))
                off += e.part.numel
            self.backend.reduce_mean_to_(flat, owner)
            if owner == self.rank:
                off = 0
                for e in dense:
                    g = self._params[e.part.var_name].grad
                    e.part.view(g).copy_(flat[off:off + e.part.numel].view(e.part.view(g).shape))
                    off += e.part.numel

    def _reduce_ps_sparse(self):
        self._touched_rows = {}
        by_var: Dict[str, list] = {}
        for e in self.plan.ps_entries.values():
            if e.part.sparse:
                by_var.setdefault(e.part.var_name, []).append(e)
        for vname, entries in by_var.items():
            p = self._params[vname]
            idx, val = self._rows_of(p)
            gi, gv = self.backend.all_gather_rows(idx, val)
            gv = gv / self.world_size
            self._touched_rows[vname] = torch.unique(gi)
            owned = [e for e in entries if e.owner == self.rank]
            if not owned:
                p.grad = None
                continue
            # keep only rows of shards this rank owns; the rest is the other owners' business
            keep = torch.zeros_like(gi, dtype=torch.bool)
            for e in owned:
                lo = 0 if e.part.part_index is None else e.part.offset
                hi = p.shape[0] if e.part.part_index is None else e.part.offset + e.part.size
                keep |= (gi >= lo) & (gi < hi)
            p.grad = torch.sparse_coo_tensor(gi[keep].unsqueeze(0), gv[keep], p.shape).coalesce()

    # -- step 5: local optimizer -----------------------------------------------------
    def _clip(self, train_op):
        if not train_op.clip_global_norm:
            return
        max_norm, params = train_op.clip_global_norm
        ids = {id(p) for p in params}
        if self.device.type == "cuda":
            return self._clip_on_device(max_norm, ids)
        sq = torch.zeros((), dtype=torch.float64, device=self.device)
        touched = []
        for t in self._targets:
            if id(t.full_param) not in ids or t.full_param.grad is None:
                continue
            g = t.grad_view(self._dense_grad(t.full_param))
            replicated = t.part is None or t.var_name not in {e.part.var_name for e in self.plan.ps_entries.values()}
            weight = 1.0 / self.world_size if (replicated and self.world_size > 1) else 1.0
            sq += weight * g.double().pow(2).sum()
            touched.append(g)
        total = self.backend.all_reduce_scalar(float(sq), "sum") if self.world_size > 1 else float(sq)
        norm = total ** 0.5
        if norm > max_norm:
            for g in touched:
                g.mul_(max_norm / (norm + 1e-6))

    def _clip_on_device(self, max_norm, ids):
        """Global-norm clip with the sum-of-squares and scale kernels: the norm never visits the host."""
        from autodist_b200.ops.functional import clip_by_global_norm_
        ps_vars = {e.part.var_name for e in self.plan.ps_entries.values()}
        grads, weights = [], []
        for t in self._targets:
            if id(t.full_param) not in ids or t.full_param.grad is None:
                continue
            g = t.grad_view(self._dense_grad(t.full_param))
            if g.dtype != torch.float32 or not g.is_contiguous():
                continue
            replicated = t.part is None or t.var_name not in ps_vars
            grads.append(g)
            weights.append(1.0 / self.world_size if (replicated and self.world_size > 1) else 1.0)
        if not grads:
            return
        reduce = None
        if self.world_size > 1:
            import torch.distributed as dist
            reduce = lambda acc: dist.all_reduce(acc, group=getattr(self.backend, "group", None))   # noqa: E731
        clip_by_global_norm_(grads, max_norm, weights, reduce)

    def _apply_local(self, train_op):
        info, local, group_map = self._local_optimizers[train_op.optimizer_index]
        if local is None:
            return
        # Follow learning-rate schedules etc. that the user applies to the captured optimizer.
        for lg, gi in zip(local.param_groups, group_map):
            for k, v in info.optimizer.param_groups[gi].items():
                if k != "params":
                    lg[k] = v
        sparse_ok = op_info.supports_sparse_rows(local)
        for t in self._targets:
            g = t.full_param.grad
            if t.param is t.full_param:
                if g is not None and g.is_sparse and not sparse_ok:
                    t.full_param.grad = g.to_dense()
                continue
            if g is None:
                t.param.grad = None
            elif g.is_sparse and sparse_ok and t.part.axis == 0:
                # rows of this shard only, re-based to the shard: the table's gradient is never made dense
                g = g.coalesce()
                rows = g.indices()[0]
                sel = (rows >= t.part.offset) & (rows < t.part.offset + t.part.size)
                t.param.grad = torch.sparse_coo_tensor((rows[sel] - t.part.offset).unsqueeze(0), g.values()[sel],
                                                       t.param.shape).coalesce()
            elif g.is_sparse:
                dense = g.to_dense()
                t.full_param.grad = dense
                t.param.grad = t.grad_view(dense)
            else:
                t.param.grad = t.grad_view(g)
        local.step()

    # -- relaxed parameter-server modes (called from the owner's server thread) -------------
    def _apply_pushed(self, op_index, grads):
        info, local, group_map, targets = self._ps_local[op_index]
        for lg, gi in zip(local.param_groups, group_map):
            for k, v in info.optimizer.param_groups[gi].items():
                if k != "params":
                    lg[k] = v
        for t in targets:
            g = grads.get(t.part.part_name)
            t.param.grad = None if g is None else torch.from_numpy(g).to(t.param.device).view_as(t.param)
        local.step()

    def _owned_values(self):
        out = {}
        for _, _, _, targets in self._ps_local.values():
            for t in targets:
                out[t.part.part_name] = t.param.detach().cpu().contiguous().numpy()
        return out

    # -- step 6: owners publish -------------------------------------------------------
    def _row_publish_vars(self):
        """Row-sparse parameter-server variables whose optimizer changes only the rows that received a gradient
        (sparse-capable optimizers): owners publish those rows instead of their whole shard."""
        cached = getattr(self, "_row_publish_cache", None)
        if cached is not None:
            return cached
        sparse_ok_params = set()
        for info, local, _ in self._local_optimizers:
            if op_info.supports_sparse_rows(info.optimizer):
                for g in info.optimizer.param_groups:
                    sparse_ok_params.update(id(p) for p in g["params"])
        by_var: Dict[str, list] = {}
        for e in self.plan.ps_entries.values():
            by_var.setdefault(e.part.var_name, []).append(e)
        out = set()
        for vname, entries in by_var.items():
            p = self._params[vname]
            if id(p) in sparse_ok_params and p.dim() >= 1 and all(
                    e.part.sparse and (e.part.part_index is None or e.part.axis == 0) for e in entries):
                out.add(vname)
        self._row_publish_cache = out
        return out

    def _publish_rows(self, vname):
        """Every rank knows the rows touched this step (the gathered indices); each row's owner contributes its new
        value to a sum over ranks, everybody else contributes zero."""
        rows = getattr(self, "_touched_rows", {}).get(vname)
        if rows is None or rows.numel() == 0:
            return
        p = self._params[vname]
        mine = torch.zeros_like(rows, dtype=torch.bool)
        for e in self.plan.ps_entries.values():
            if e.part.var_name == vname and e.owner == self.rank:
                lo = 0 if e.part.part_index is None else e.part.offset
                hi = p.shape[0] if e.part.part_index is None else e.part.offset + e.part.size
                mine |= (rows >= lo) & (rows < hi)
        vals = p.data[rows]
        vals[~mine] = 0
        self.backend.all_reduce_sum_(vals)
        p.data[rows] = vals

    def _publish_ps(self):
        by_rows = self._row_publish_vars()
        for vname in sorted(by_rows):
            self._publish_rows(vname)
        for owner, entries in sorted(self.plan.ps_by_owner().items()):
            entries = [e for e in entries if e.part.var_name not in by_rows]
            if not entries:
                continue
            numel = sum(e.part.numel for e in entries)
            dtype = self._params[entries[0].part.var_name].dtype
            flat = self._buffer(("pub", owner), numel, dtype)
            if owner == self.rank:
                off = 0
                for e in entries:
                    src = e.part.view(self._params[e.part.var_name].data)
                    flat[off:off + e.part.numel].view(src.shape).copy_(src)
                    off += e.part.numel
            self.backend.broadcast_(flat, owner)
            if owner != self.rank:
                off = 0
                for e in entries:
                    dst = e.part.view(self._params[e.part.var_name].data)
                    dst.copy_(flat[off:off + e.part.numel].view(dst.shape))
                    off += e.part.numel

    # ------------------------------------------------------------------ state for checkpoints
    def variable_value(self, name):
        self.before_read()
        return self._params[name].detach()

    def optimizer_slots(self):
        """``"<var op name>/<slot>" -> full-shaped tensor`` with shards merged across owners."""
        self.before_read()
        out = {}
        for info, local, _ in self._local_optimizers:
            names = op_info.slot_names(info.cls)
            full: Dict[str, torch.Tensor] = {}
            if local is not None:
                for t in self._targets:
                    st = local.state.get(t.param)
                    if not st:
                        continue
                    for slot in names:
                        if slot not in st or st[slot] is None or not torch.is_tensor(st[slot]):
                            continue
                        key = f"{t.var_name[:-2]}/{slot}"
                        if key not in full:
                            full[key] = torch.zeros_like(t.full_param.data)
                        (full[key] if t.part is None else t.part.view(full[key])).copy_(st[slot])
                    if "step" in st:
                        full.setdefault(f"{t.var_name[:-2]}/step", torch.as_tensor(float(st["step"])))
            # merge across owners: every slot key exists on the ranks that own a piece of it
            if self.world_size > 1 and self.plan.ps_entries:
                keys = sorted({f"{e.part.var_name[:-2]}/{s}" for e in self.plan.ps_entries.values() for s in names})
                for key in keys:
                    vname = key.rsplit("/", 1)[0] + ":0"
                    buf = full.get(key)
                    if buf is None:
                        buf = torch.zeros_like(self._params[vname].data)
                    has = self.backend.all_reduce_scalar(1.0 if key in full else 0.0, "sum")
                    if has == 0:
                        continue
                    buf = buf.clone()
                    import torch.distributed as dist
                    dist.all_reduce(buf)
                    full[key] = buf
            out.update(full)
        return out

    def load_optimizer_slots(self, slots, default_step=0):
        for info, local, _ in self._local_optimizers:
            if local is None:
                continue
            names = op_info.slot_names(info.cls)
            members = {id(p) for g in local.param_groups for p in g["params"]}
            for t in self._targets:
                if id(t.param) not in members:
                    continue
                loaded = {}
                for slot in names:
                    key = f"{t.var_name[:-2]}/{slot}"
                    if key in slots:
                        src = slots[key].to(self.device)
                        loaded[slot] = (src if t.part is None else t.part.view(src)).clone()
                if not loaded:
                    continue
                st = local.state[t.param]
                st.update(loaded)
                # The writer only knows the step counters of the parts it owned; the rest took as many steps.
                step = slots.get(f"{t.var_name[:-2]}/step", default_step)
                st["step"] = torch.as_tensor(float(step))

    def close(self):
        if self._async is not None:
            self._async.close()
        # A lazily refreshed parameter-server variable is pulled by a collective the next time any rank reads it. A
        # rank that is done takes part in that last pull here, so that a peer which still fetches variables after
        # its final step (the chief printing them, a checkpoint) is not left waiting for it.
        if self.world_size > 1 and self._pending_pull:
            try:
                self.before_read()
            except Exception as e:  # the peers may already be gone
                logging.debug("final parameter pull skipped: %s", e)
                self._pending_pull = False
