"""Step engine for models that run on the hand-written sm_100a kernels.

Chosen on CUDA devices when the captured graph is one leaf module that
implements ``materialize`` / ``fused_forward_backward`` (e.g.
``models.bert.BertPretrainer``). Differences to the generic ``StepEngine``:

* parameters, their bf16 compute copies, gradients and optimizer slots are flat
  buffers; the gradient buffer is symmetric memory mapped by every rank;
* all-reduce buckets are *flights*: as the backward pass reports a finished
  range of the flat gradient buffer, its all-reduce kernel (``comm.cu``: cast +
  error feedback + two-shot mean over peer memory, NVLS when available) is
  launched on a communication stream, followed by the fused optimizer kernel for
  that range, while the compute stream continues with earlier layers;
* the whole step (input staging excluded) can be captured once into a CUDA graph
  and replayed, because every kernel argument (flags, epochs, step counter,
  learning rate) lives in device memory.

Strategies this engine executes natively: all-reduce buckets with
``NoneCompressor`` / ``HorovodCompressor`` / ``HorovodCompressorEF``
(``allreduce_kernel``); parameter-server variables and shards with GPU owners as
owned segments of the flat buffers (``reduce_scatter_update``: reduce to the
owner, optimizer on the owner's state, parameter write-back to every rank); and
row-sparse variables sharded one shard per rank, which are not replicated at all
(``embedding_gather_peers`` for lookups, ``sparse_scatter_add`` into the owners'
shards, owner-side update). Anything else (PowerSGD, relaxed parameter-server
gates, clipping, partition axes other than 0) runs on the generic engine over
NCCL, which is also the measured baseline (``AUTODIST_COMM=nccl``).
"""
import os

import torch
import torch.distributed as dist

from autodist_b200.const import ENV
from autodist_b200.kernel.synchronization.compressor import wire_dtype
from autodist_b200.parallel.engine import StepEngine
from autodist_b200.utils import logging, nvtx

WIRE = {None: 0, torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
PowerSGD_SEED = 1905_13727        # seed base of the initial Q factors (kernel/synchronization/compressor.py uses the same)


def _fused_module(graph_item):
    mods = [graph_item.root.get_submodule(n.target) for n in graph_item.tracer.graph.nodes if n.op == "call_module"]
    mods = [m for m in mods if hasattr(m, "fused_forward_backward")]
    if len(mods) != 1:
        return None
    m = mods[0]
    own = {id(p) for p in m.parameters()}
    for _, p in graph_item.named_parameters():
        if p.requires_grad and id(p) not in own:
            return None
    return m


def make_engine(graph_item, plan, backend, device):
    module = _fused_module(graph_item)
    fused_comm = ENV.AUTODIST_COMM.val != "nccl"
    if module is not None and fused_comm and FusedStepEngine.supports(graph_item, plan, module):
        return FusedStepEngine(graph_item, plan, backend, device, module)
    if module is not None:
        logging.info("fused model on the generic engine (communication through %s)", backend.name)
        return GenericFusedModelEngine(graph_item, plan, backend, device, module)
    if fused_comm and FlatAutogradEngine.supports_autograd(graph_item, plan):
        return FlatAutogradEngine(graph_item, plan, backend, device)
    return StepEngine(graph_item, plan, backend, device)


class GenericFusedModelEngine(StepEngine):
    """Fused compute kernels, generic synchronisation (torch.distributed collectives + torch optimizers):
    the NCCL baseline for the same model."""

    def __init__(self, graph_item, plan, backend, device, module):
        self.module = module
        super().__init__(graph_item, plan, backend, device)

    def _move_to_device(self):
        self.module.materialize(self.device)

    def _share_initial_values(self):
        if self.world_size > 1:
            self.backend.broadcast_(self.module.flat.master, 0)
        self.module.flat.refresh_bf16()

    def before_read(self):
        if self._pending_pull:
            super().before_read()
            self.module.flat.refresh_bf16()      # lazily pulled parameter-server values reach the compute copy too

    def train_step(self, train_op, nodes, feeds):
        self.before_read()
        all_nodes = list(nodes)
        if train_op.loss_node not in all_nodes:
            all_nodes.append(train_op.loss_node)
        fl = self.module.flat
        for name, p in zip(fl.names, fl.params):
            p.grad = fl.g[name]          # the generic sparse paths replace .grad; the model always writes the flat views
        values = self.forward(all_nodes, feeds, grad=True)
        self.sync_and_update(train_op)
        self.module.flat.refresh_bf16()
        self.global_step += 1
        return [v.detach() if isinstance(v, torch.Tensor) else v for v in values[:len(nodes)]]


class SymmetricArena:
    """Symmetric buffers of one process group plus the flag words of the in-kernel barriers."""

    def __init__(self, group, device, rank, world):
        import torch.distributed._symmetric_memory as symm
        self.symm = symm
        self.group = group
        self.device = device
        self.rank, self.world = rank, world
        from autodist_b200 import ops
        self.E = ops.ext(required=True)
        nflags = self.E.MAX_COMM_BLOCKS * 8
        self.flags, self.flag_ptrs, _ = self.alloc(nflags, torch.int32)
        self.flags.zero_()
        self.epochs = torch.zeros(self.E.MAX_COMM_BLOCKS + 8, dtype=torch.int32, device=device)
        # a second, independent set of flags for kernels issued from another stream (barrier epochs are per channel)
        self.flags_b, self.flag_ptrs_b, _ = self.alloc(nflags, torch.int32)
        self.flags_b.zero_()
        self.epochs_b = torch.zeros(self.E.MAX_COMM_BLOCKS + 8, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        self.timeout_s = float(os.environ.get("AUTODIST_KERNEL_TIMEOUT", "20"))
        torch.cuda.synchronize()
        dist.barrier(group=group)

    GUARD_BYTES = 256      # canary words before and after every symmetric buffer (keeps 256-byte alignment)

    def alloc(self, numel, dtype):
        """(local tensor, int64 device tensor of every rank's address, multicast address or 0).

        The buffer sits between two guard regions filled with a pattern; ``check_canaries`` tells whether this rank
        or a peer wrote outside a buffer."""
        item = torch.empty((), dtype=dtype).element_size()
        guard = self.GUARD_BYTES // item
        raw = self.symm.empty(numel + 2 * guard, dtype=dtype, device=self.device)
        hdl = self.symm.rendezvous(raw, self.group.group_name if hasattr(self.group, "group_name") else self.group)
        words = raw.view(torch.uint8)
        words[:self.GUARD_BYTES] = self.CANARY
        words[self.GUARD_BYTES + numel * item:] = self.CANARY
        if not hasattr(self, "_guards"):
            self._guards = []
        self._guards.append((words, numel * item))
        t = raw[guard:guard + numel]
        ptrs = torch.tensor([int(p) + self.GUARD_BYTES for p in hdl.buffer_ptrs], dtype=torch.int64, device=self.device)
        mc = 0
        if os.environ.get("AUTODIST_NVLS", "1") != "0":
            try:
                mc = int(hdl.multicast_ptr or 0)
            except Exception:  # no multicast support on this fabric / build
                mc = 0
        return t, ptrs, (mc + self.GUARD_BYTES if mc else 0)

    CANARY = 0xA5

    def check_canaries(self):
        """Raise if any guard byte around a symmetric buffer of this rank changed (an out-of-bounds write, local or
        from a peer). Synchronises the device; meant for tests and debugging, not for the step loop."""
        torch.cuda.synchronize()
        for i, (words, nbytes) in enumerate(getattr(self, "_guards", [])):
            lo, hi = words[:self.GUARD_BYTES], words[self.GUARD_BYTES + nbytes:]
            if not (bool((lo == self.CANARY).all()) and bool((hi == self.CANARY).all())):
                raise RuntimeError(f"rank {self.rank}: guard words of symmetric buffer {i} were overwritten")

    def ctx(self, channel=0):
        if channel:
            return (self.flag_ptrs_b, self.epochs_b, self.error, self.rank, self.world, self.timeout_s)
        return (self.flag_ptrs, self.epochs, self.error, self.rank, self.world, self.timeout_s)

    def reset_error(self):
        """Clear a recorded time-out and the words of the in-rank block barrier: a barrier that gave up leaves its arrival
        count behind, which would make the next launch on that channel miscount."""
        torch.cuda.synchronize()
        self.error.zero_()
        n = self.E.MAX_COMM_BLOCKS
        self.epochs[n:n + 2].zero_()
        self.epochs_b[n:n + 2].zero_()

    def check(self):
        code = int(self.error.item())
        if code:
            if code in (301, 302):
                raise RuntimeError(f"rank {self.rank}: a row id outside the sharded table reached the "
                                   f"{'scatter-add' if code == 301 else 'gather'} kernel (code {code}); the row was skipped")
            raise RuntimeError(f"rank {self.rank}: a communication kernel gave up waiting for a peer (code {code})")


def row_shard_candidates(item, plan, hand_scheduled):
    """``{variable name: parameter}`` of the row-sparse tables that are kept as one shard per rank instead of replicated.

    A table qualifies when its module reads it through ``ops.functional.sparse_lookup`` (it lists the parameter in
    ``sparse_lookup_parameters()``), it is fp32 ``[V, H]`` with ``H`` a multiple of 8, and - with more than one rank -
    the plan splits it along axis 0 into one part per rank, part ``i`` owned by rank ``i`` (what ``Parallax`` and
    ``PartitionedPS(num_shards=<gpus>)`` with ``reduction_devices="gpu"`` produce). The scatter-add into owner shards
    uses floating-point atomics, whose order of addition varies from run to run; ``AUTODIST_DETERMINISTIC=1`` (or
    ``AUTODIST_SPARSE_ROWS=0``) keeps such tables replicated and their gradients on the dense paths."""
    if os.environ.get("AUTODIST_SPARSE_ROWS", "1") == "0" or os.environ.get("AUTODIST_DETERMINISTIC", "0") == "1":
        return {}
    declared = set()
    for m in item.root.modules():
        declared |= {id(p) for p in getattr(m, "sparse_lookup_parameters", lambda: [])()}
    by_var = {}
    for e in plan.ps_entries.values():
        by_var.setdefault(e.part.var_name, []).append(e)
    out = {}
    world = plan.replica.world_size
    for var_name, p in item.named_parameters():
        var = item.variables.get(var_name)
        if var is None or not var.sparse_grad or id(p) not in declared or not p.requires_grad:
            continue
        if world == 1 and hand_scheduled:
            continue      # a hand-scheduled model keeps its tables in the flat buffers: nothing to gain on one rank
        if p.dim() != 2 or p.shape[1] % 8 or p.dtype != torch.float32 or p.shape[0] < world:
            continue
        if world > 1:
            entries = sorted(by_var.get(var_name, []), key=lambda e: e.part.offset)
            q, rem = divmod(p.shape[0], world)
            if len(entries) != world or not all(e.part.sparse and e.gate == "sync" for e in entries) \
                    or [e.owner for e in entries] != list(range(world)) \
                    or [e.part.size for e in entries] != [q + (1 if i < rem else 0) for i in range(world)]:
                continue
        out[var_name] = p
    return out


class LocalArena:
    """Stand-in for ``SymmetricArena`` in a single-process job: plain device buffers with the same ``alloc`` / ``ctx`` face,
    so that the row-sharded table kernels (one shard, no peers, no barriers) run unchanged on one GPU."""

    def __init__(self, device):
        from autodist_b200 import ops
        self.E = ops.ext(required=True)
        self.device = device
        self.rank, self.world = 0, 1
        self.flags = torch.zeros(self.E.MAX_COMM_BLOCKS * 8, dtype=torch.int32, device=device)
        self.flag_ptrs = torch.tensor([self.flags.data_ptr()], dtype=torch.int64, device=device)
        self.epochs = torch.zeros(self.E.MAX_COMM_BLOCKS + 8, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        self.timeout_s = 1.0

    def alloc(self, numel, dtype):
        t = torch.zeros(numel, dtype=dtype, device=self.device)
        return t, torch.tensor([t.data_ptr()], dtype=torch.int64, device=self.device), 0

    def ctx(self, channel=0):
        return (self.flag_ptrs, self.epochs, self.error, 0, 1, self.timeout_s)

    def check(self):
        code = int(self.error.item())
        if code:
            raise RuntimeError(f"a row id outside the table reached the sharded-table kernels (code {code})")


class ShardedRows:
    """A row-sparse ``[V, H]`` variable split along axis 0 into one shard per rank (rank ``i`` owns block ``i``) and never
    replicated: lookups gather rows from the owners inside the kernel (``embedding_gather_peers``), gradient rows are added
    straight into the owners' fp32 shards (``sparse_scatter_add``), and after the last push of a step every owner updates
    its shard. The reference reaches the same placement with a partitioned ``embedding_lookup`` over variables on the
    parameter servers (``autodist/kernel/partitioner.py:660-684``, ``examples/lm1b/language_model.py:66``).

    Step protocol (all kernels on the compute stream, flag channel 1): the first lookup of a step meets the peers first (the
    owners' updates of the previous step are complete); pushes carry no barrier; ``finish`` meets the peers once (every
    rank's rows have landed), updates and clears. Optimizers that leave untouched rows unchanged (SGD without momentum or
    weight decay, Adagrad without weight decay) update only the rows whose flag the pushes raised; others sweep the shard."""

    def __init__(self, engine, var_name, param, full_fp32, arena):
        self.engine, self.var, self.param, self.arena = engine, var_name, param, arena
        world, rank = arena.world, arena.rank
        self.V, self.H = int(full_fp32.shape[0]), int(full_fp32.numel() // full_fp32.shape[0])
        q, rem = divmod(self.V, world)
        self.rows = q + (1 if rank < rem else 0)
        self.off = rank * q + min(rank, rem)
        cap = q + 1
        dev = engine.device
        self.shard16, self.s16ptrs, _ = arena.alloc(cap * self.H, torch.bfloat16)
        self.grad32, self.g32ptrs, _ = arena.alloc(cap * self.H, torch.float32)
        self.flags8, self.f8ptrs, _ = arena.alloc((cap + 15) // 16 * 16, torch.uint8)
        self.shard16.zero_(); self.grad32.zero_(); self.flags8.zero_()
        self.master = full_fp32.reshape(self.V, self.H)[self.off:self.off + self.rows].reshape(-1).to(dev, torch.float32).clone()
        self.shard16[:self.rows * self.H].copy_(self.master)
        kind = engine.opt_kind
        self.s1 = torch.zeros_like(self.master) if engine._needs_slot1() else None
        self.s2 = torch.zeros_like(self.master) if kind in ("Adam", "AdamW") else None
        if kind == "Adagrad":
            self.s1.fill_(float(engine.opt_info.optimizer.param_groups[0].get("initial_accumulator_value", 0.0)))
        g = engine.opt_info.optimizer.param_groups[0]
        plain = float(g.get("weight_decay", 0.0)) == 0.0
        self.flagged = os.environ.get("AUTODIST_SPARSE_FLAGGED", "1") == "1" and plain and (
            kind == "Adagrad" or (kind == "SGD" and float(g.get("momentum", 0.0)) == 0.0))
        self.blocks = 32

    # -- forward / backward ------------------------------------------------------------------------------------------
    def lookup(self, ids):
        eng = self.engine
        ids = ids.reshape(-1).contiguous()
        out = torch.empty(ids.numel(), self.H, dtype=torch.bfloat16, device=eng.device)
        first = eng._rows_sync_pending and self.arena.world > 1
        eng._rows_sync_pending = False
        eng.E.embedding_gather_peers(*self.arena.ctx(1), self.s16ptrs, ids, out, self.V, 1 if first else 0, self.blocks)
        return out

    def push(self, ids, rows):
        """Add ``rows`` (bf16 or fp32 ``[n, H]``, this replica's gradient of the looked-up rows) into the owners' shards."""
        eng = self.engine
        ids = ids.reshape(-1).contiguous()
        rows = rows.reshape(ids.numel(), self.H)
        if rows.dtype not in (torch.bfloat16, torch.float32):
            rows = rows.float()
        eng.E.sparse_scatter_add(*self.arena.ctx(1), self.g32ptrs, self.f8ptrs if self.flagged else None, ids, rows.contiguous(), self.V,
                                 1.0 / self.arena.world, 0, self.blocks)
        eng._rows_dirty = True

    def update(self):
        """Owner-side optimizer step on this rank's shard (after the step's barrier), then clear what the pushes wrote."""
        eng = self.engine
        g = eng.opt_info.optimizer.param_groups[0]
        n = self.rows * self.H
        if self.flagged:
            kind = {"SGD": 0, "Adagrad": 2}[eng.opt_kind]
            eng.E.flagged_rows_update(self.master, self.s1, self.s2, self.shard16, self.grad32, self.flags8, self.rows, self.H, kind, eng.lr,
                                      0.0, 0.0, float(g.get("eps", 1e-10)), None)
            return
        eng._apply_optimizer(self.master, self.grad32[:n], self.s1, self.s2, self.shard16[:n])
        self.grad32.zero_()

    # -- state -------------------------------------------------------------------------------------------------------
    def gather(self, local_flat):
        """Full ``[V, H]`` tensor from every owner's rows (checkpoints, variable fetches)."""
        world = self.arena.world
        if world == 1:
            return local_flat[:self.rows * self.H].view(self.V, self.H).clone()
        cap = self.V // world + 1
        pad = torch.zeros(cap * self.H, dtype=torch.float32, device=self.engine.device)
        pad[:local_flat.numel()].copy_(local_flat)
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=self.engine.backend.group)
        q, rem = divmod(self.V, world)
        rows = [q + (1 if i < rem else 0) for i in range(world)]
        return torch.cat([parts[i][:rows[i] * self.H] for i in range(world)]).view(self.V, self.H)

    def load(self, full_fp32):
        """Re-slice this rank's rows out of the full table (restore)."""
        lo, hi = self.off, self.off + self.rows
        self.master.copy_(full_fp32.reshape(self.V, self.H)[lo:hi].reshape(-1))
        self.shard16[:self.rows * self.H].copy_(self.master)

    def load_slots(self, slot1=None, slot2=None):
        lo, hi = self.off, self.off + self.rows
        for own, full in ((self.s1, slot1), (self.s2, slot2)):
            if own is not None and full is not None:
                own.copy_(full.reshape(self.V, self.H)[lo:hi].reshape(-1))


class FusedStepEngine(StepEngine):
    @staticmethod
    def supports(graph_item, plan, module):
        if len(graph_item.optimizers) != 1:
            return False
        if module is not None and any(op.clip_global_norm for op in graph_item.train_ops):
            return False      # the hand-scheduled models fuse reduction and update per flight: no place for a global norm
        if type(graph_item.optimizers[0].optimizer).__name__ not in ("Adam", "AdamW", "SGD", "Adagrad"):
            return False
        if len(graph_item.optimizers[0].optimizer.param_groups) > 1 and (plan.ps_entries or plan.sparse_all_reduce):
            # several parameter groups (their own learning rate, weight decay, ...) are applied range by range of the flat
            # buffer after an all-reduce; the owner-side update kernels take one set of hyper-parameters per launch
            return False
        if plan.replica.world_size > 1:
            # A variable split into all-reduce parts (PartitionedAR, RandomAxisPartitionAR: any axis) is reduced as the one
            # range it occupies in the flat buffer: the mean is element-wise, so reducing the parts separately or together
            # gives the same values as long as all parts of a variable use one compressor.
            compressor_of = {}
            for b in plan.ordered_buckets():
                if b.compressor_type == "PowerSGDCompressor" and (max(1, b.power_sgd_rank or 1) > 4 or any(
                        p.part_index is not None for p in b.parts)):
                    return False
                for p in b.parts:
                    if compressor_of.setdefault(p.var_name, b.compressor_type) != b.compressor_type:
                        return False
            for e in plan.ps_entries.values():
                if e.part.part_index is not None and e.part.axis != 0:
                    return False
            if plan.gate_mode != "sync":
                # Bounded staleness / asynchronous updates with GPU owners: every worker applies its own gradient to the
                # owner's copy as a reduction over NVLink, which is only order-independent for plain SGD; there is no
                # lock-step collective in such a step, so all-reduce buckets cannot be mixed in. Anything else keeps
                # the host-side service of the generic engine.
                g = graph_item.optimizers[0].optimizer.param_groups[0]
                plain_sgd = type(graph_item.optimizers[0].optimizer).__name__ == "SGD" and not g.get("momentum", 0) \
                    and not g.get("weight_decay", 0)
                if not plain_sgd or plan.ar_buckets or plan.sparse_all_reduce or any(e.gate == "sync" for e in plan.ps_entries.values()):
                    return False
        return True

    def __init__(self, graph_item, plan, backend, device, module):
        self.module = module
        self.item = graph_item
        self.plan = plan
        self.backend = backend
        self.device = torch.device(device)
        self.rank, self.world_size = plan.replica.rank, plan.replica.world_size
        self.global_step = 0
        self._compiled = {}
        self._async = None
        self._pending_pull = False
        from autodist_b200 import ops
        self.E = ops.ext(required=True)
        self.arena = None
        grad_alloc = None
        if self.world_size > 1:
            self.arena = SymmetricArena(backend.group, self.device, self.rank, self.world_size)
            self._grad_sym = {}

            def grad_alloc(n):
                t, ptrs, mc = self.arena.alloc(n, torch.float32)
                t.zero_()
                self._grad_sym = {"ptrs": ptrs, "mc": mc}
                return t
        self._params = {name: p for name, p in graph_item.named_parameters()}
        self.sharded_rows = {}
        self._rows_sync_pending, self._rows_dirty = True, False
        row_sharded = self._row_shard_candidates()
        master_alloc = p16_alloc = None
        self._p32_sym = self._p16_sym = None
        self._p32_mc = self._p16_mc = 0
        if self.world_size > 1 and any(e.part.var_name not in row_sharded for e in plan.ps_entries.values()):
            # owners write updated parameters straight into every rank's copies: those live in symmetric memory too
            def master_alloc(n):
                t, ptrs, mc = self.arena.alloc(n, torch.float32)
                t.zero_()
                self._p32_sym, self._p32_mc = ptrs, mc
                return t

            def p16_alloc(n):
                t, ptrs, mc = self.arena.alloc(n, torch.bfloat16)
                t.zero_()
                self._p16_sym, self._p16_mc = ptrs, mc
                return t
        if isinstance(module, _AutogradModel):
            # tables that are never replicated stay out of the flat buffers: no full-size gradient, compute copy or slots
            self.flat = module.materialize(self.device, grad_alloc, master_alloc, p16_alloc, exclude={id(p) for p in row_sharded.values()})
        else:
            self.flat = module.materialize(self.device, grad_alloc, master_alloc, p16_alloc)
        if self.world_size > 1:
            backend.broadcast_(self.flat.master, 0)
        self.flat.refresh_bf16()
        self._setup_optimizer()
        self._setup_sharded_rows(row_sharded)
        self._setup_flights()
        self.comm_stream = torch.cuda.Stream(device=self.device)
        self._ready_event = torch.cuda.Event()
        self._done_event = torch.cuda.Event()
        self._graph = None
        self._static_feeds = None
        self._use_graph = os.environ.get("AUTODIST_CUDA_GRAPH", "1") != "0"
        self._warm_steps = 0
        self.launches_per_step = 0
        self.graph_kernels = 0
        # AUTODIST_FLIGHT_TIMING=1: CUDA events around every flight of a step (read them with `flight_report`).
        # Timed events cannot be recorded into a CUDA graph, so the step runs as eager launches while this is on.
        self._flight_log = [] if os.environ.get("AUTODIST_FLIGHT_TIMING", "0") == "1" else None
        self._step_start = None
        module.grad_ready = self._on_grad_ready
        if self.world_size > 1:
            torch.cuda.synchronize()
            dist.barrier(group=backend.group)

    # ------------------------------------------------------------------ optimizer state
    def _setup_optimizer(self):
        info = self.item.optimizers[0]
        self.opt_info = info
        self.opt_kind = type(info.optimizer).__name__
        n = self.flat.total
        dev = self.device
        # parameter groups: runs of the flat buffer whose parameters share a group (adjacent parameters of one group merge)
        groups = info.optimizer.param_groups
        group_of = {id(p): gi for gi, g in enumerate(groups) for p in g["params"]}
        fl = self.flat
        self._group_runs = []                       # (lo, hi, group index), ascending
        for name, p in zip(fl.names, fl.params):
            lo = fl.offsets[name]
            hi = lo + p.numel()
            gi = group_of.get(id(p), 0)
            if self._group_runs and self._group_runs[-1][2] == gi and self._group_runs[-1][1] == lo:
                self._group_runs[-1] = (self._group_runs[-1][0], hi, gi)
            else:
                self._group_runs.append((lo, hi, gi))
        self.slot1 = torch.zeros(n, dtype=torch.float32, device=dev) if self._needs_slot1() else None
        if self.opt_kind == "Adagrad":
            for lo, hi, gi in self._group_runs:
                self.slot1[lo:hi].fill_(float(groups[gi].get("initial_accumulator_value", 0.0)))
        self.slot2 = torch.zeros(n, dtype=torch.float32, device=dev) if self.opt_kind in ("Adam", "AdamW") else None
        self.lrs = torch.zeros(len(groups), dtype=torch.float32, device=dev)      # one learning rate per group, read by the kernels
        self.lr = self.lrs[0:1]
        self._lr_host = None
        self.opt_step = torch.zeros(1, dtype=torch.int64, device=dev)
        self._sync_lr()

    def _needs_slot1(self):
        return self.opt_kind != "SGD" or any(g.get("momentum", 0) != 0 for g in self.opt_info.optimizer.param_groups)

    def _sync_lr(self):
        lrs = [float(g["lr"]) for g in self.opt_info.optimizer.param_groups]
        if lrs != self._lr_host:
            for gi, lr in enumerate(lrs):                    # device-side fills: a schedule that moves every step never syncs
                if self._lr_host is None or self._lr_host[gi] != lr:
                    self.lrs[gi:gi + 1].fill_(lr)
            self._lr_host = lrs

    def _update_range(self, lo, hi):
        """Optimizer update of the flat range [lo, hi): one launch per parameter group that has parameters in it."""
        fl = self.flat
        for glo, ghi, gi in self._group_runs:
            a, b = max(lo, glo), min(hi, ghi)
            if a < b:
                self._apply_optimizer(fl.master[a:b], fl.grad[a:b], self.slot1[a:b] if self.slot1 is not None else None,
                                      self.slot2[a:b] if self.slot2 is not None else None, fl.p16[a:b], gi)

    # ------------------------------------------------------------------ flights
    def _setup_flights(self):
        """Which compressor applies to which range of the flat gradient buffer."""
        fl = self.flat
        self.range_wire = []     # (lo, hi, wire dtype or None, error feedback?)
        self.ps_segments = []
        self._wire = self._wire_ptrs = self._residual = None
        self._psgd, self._psgd_flights = None, []
        self._relaxed = None
        if self.world_size <= 1:
            return
        need16 = False
        per_var = []
        flat_name = {self.item.name_of_parameter(p): n for n, p in zip(fl.names, fl.params)}   # "x:0" -> flat key
        self._range_key = []      # (lo, hi, collective group key, first instance key) per bucket: names the trace ranges
        psgd = []                 # (start in the flat buffers, m, n, seed of the initial Q) of every PowerSGD matrix
        self._psgd_rank = 1
        for b in self.plan.ordered_buckets():
            power = b.compressor_type == "PowerSGDCompressor"
            wd = None if b.compressor_type == "NoneCompressor" or power else wire_dtype()
            ef = b.compressor_type == "HorovodCompressorEF"
            need16 |= wd is not None
            spans = []
            rank_r = max(1, b.power_sgd_rank or 1)
            for idx, part in enumerate(b.parts):
                lo_v, hi_v = fl.offsets[flat_name[part.var_name]], fl.range_of([flat_name[part.var_name]])[1]
                spans.append((lo_v, hi_v))
                shape = b.shapes[idx]
                numel = 1
                for d in shape:
                    numel *= int(d)
                if power and len(shape) >= 2 and min(int(shape[0]), numel // int(shape[0])) > rank_r:
                    # a matrix travels as its two factors; the PowerSGD passes of the step handle it (see _finish_powersgd)
                    psgd.append((lo_v, int(shape[0]), numel // int(shape[0]), PowerSGD_SEED + idx))
                    self._psgd_rank = rank_r
                    continue
                per_var.append((lo_v, hi_v, wd, ef))
            if spans:
                self._range_key.append((min(a for a, _ in spans), max(z for _, z in spans), b.group_key,
                                        b.instance_keys[0] if b.instance_keys else 0))
        # Row-sparse variables under an all-reduce strategy: this model writes their gradient densely into the flat
        # buffer, so the mean over replicas is the same all-reduce, uncompressed.
        for part, _, _ in self.plan.sparse_all_reduce:
            per_var.append((fl.offsets[flat_name[part.var_name]], fl.range_of([flat_name[part.var_name]])[1], None, False))
        per_var = sorted(set(per_var))          # the parts of a partitioned variable name the same range once
        for lo, hi, wd, ef in per_var:
            if self.range_wire and self.range_wire[-1][1] == lo and self.range_wire[-1][2:4] == (wd, ef):
                self.range_wire[-1] = (self.range_wire[-1][0], hi, wd, ef, None)
            else:
                self.range_wire.append((lo, hi, wd, ef, None))
        if need16:
            self._wire, self._wire_ptrs, self._wire_mc = self.arena.alloc(fl.total, wire_dtype())
            self._residual = torch.zeros(fl.total, dtype=torch.float32, device=self.device)
        self._setup_ps_segments(flat_name)
        self._setup_powersgd(psgd)
        self._setup_relaxed()

    # ---- relaxed parameter server on GPUs (bounded staleness / asynchronous): push, gate, pull -------------------------------
    def _setup_relaxed(self):
        """``sync=False`` or ``staleness > 0`` with GPU owners (reference: token queues of capacity ``staleness`` and unaggregated
        updates, ``autodist/kernel/synchronization/ps_synchronizer.py:261-262,388-458``). Each flight pushes this worker's
        gradient into the owners' fp32 copies (``relaxed_push_sgd``: vector reductions over NVLink); at the end of the step
        the worker publishes its step and - under bounded staleness - waits until it is at most ``staleness`` steps ahead of
        the slowest peer (``staleness_gate``, a bounded wait that reports ``200 + peer``), then refreshes its copies from the
        owners (``relaxed_pull``). Nothing in such a step is a collective, so a slow worker delays nobody beyond the bound."""
        self._relaxed = None
        if self.world_size <= 1 or self.plan.gate_mode == "sync" or not self.ps_segments:
            return
        dev = self.device
        t = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)        # noqa: E731
        clocks, cptrs, _ = self.arena.alloc(8, torch.int32)
        clocks.zero_()
        self._relaxed = {"staleness": int(self.plan.staleness) if self.plan.gate_mode == "stale" else -1, "clocks": clocks, "cptrs": cptrs,
                         "max_lead": torch.zeros(1, dtype=torch.int32, device=dev), "tables": {}, "t": t}
        self.arena.timeout_s = float(os.environ.get("AUTODIST_GATE_TIMEOUT", str(self.arena.timeout_s)))
        torch.cuda.synchronize()
        dist.barrier(group=self.backend.group)

    def _relaxed_table(self, lo, hi):
        tabs = self._relaxed["tables"]
        if (lo, hi) not in tabs:
            inside = [(st, ln, ow) for st, ln, ow in self.ps_segments if st >= lo and st + ln <= hi]
            prefix = [0]
            for _, ln, _ in inside:
                prefix.append(prefix[-1] + ln)
            t = self._relaxed["t"]
            tabs[(lo, hi)] = (t([x[0] for x in inside] or [0]), t([x[1] for x in inside] or [0]), t([x[2] for x in inside] or [0]), t(prefix),
                              prefix[-1]) if inside else None
        return tabs[(lo, hi)]

    def _relaxed_push(self, lo, hi):
        tab = self._relaxed_table(lo, hi)
        if tab is None:
            return
        starts, lens, owners, prefix, total = tab
        blocks = max(8, min(self.E.MAX_COMM_BLOCKS, total // (4 * 512 * 4) + 1))
        self.E.relaxed_push_sgd(self._p32_sym, self.flat.grad, starts, lens, owners, prefix, self.lr, 1.0, blocks)

    def _finish_relaxed(self):
        r = self._relaxed
        if not r:
            return
        compute = torch.cuda.current_stream()
        self._ready_event.record(compute)
        self.comm_stream.wait_event(self._ready_event)
        with torch.cuda.stream(self.comm_stream):
            self.E.staleness_gate(*self.arena.ctx(), r["cptrs"], 0, r["staleness"], self.opt_step, r["max_lead"])
            tab = self._relaxed_table(0, self.flat.total)
            if tab is not None:
                starts, lens, owners, prefix, total = tab
                blocks = max(8, min(self.E.MAX_COMM_BLOCKS, total // (4 * 512 * 4) + 1))
                self.E.relaxed_pull(self._p32_sym, self.flat.master, self.flat.p16, starts, lens, owners, prefix, self.rank, blocks)

    @property
    def max_lead(self):
        """Largest number of steps this rank was ahead of the slowest peer when it passed the staleness gate."""
        return int(self._relaxed["max_lead"].item()) if self._relaxed else 0

    # ---- PowerSGD (K8): every matrix of the step in three batched passes + two all-reduces of the stacked factors -------------
    def _setup_powersgd(self, mats):
        self._psgd = None
        if not mats:
            return
        fl, dev, r = self.flat, self.device, self._psgd_rank
        mats.sort()
        p_off, q_off, rows, blks, elems = [], [], [0], [0], [0]
        pn = qn = 0
        for lo, m, n, _ in mats:
            p_off.append(pn); q_off.append(qn)
            pn += m * r; qn += n * r
            rows.append(rows[-1] + m); blks.append(blks[-1] + (n + 31) // 32); elems.append(elems[-1] + m * n)
        pn4, qn4 = (pn + 3) // 4 * 4, (qn + 3) // 4 * 4
        P, p_ptrs, p_mc = self.arena.alloc(pn4, torch.float32)
        Q, q_ptrs, q_mc = self.arena.alloc(qn4, torch.float32)
        P.zero_(); Q.zero_()
        for (lo, m, n, seed), qo in zip(mats, q_off):       # the same start as the Python compressor: N(0, 1) from a per-matrix seed
            g = torch.Generator(device="cpu").manual_seed(seed)
            Q[qo:qo + n * r].copy_(torch.randn(n, r, generator=g, dtype=torch.float32).reshape(-1))
        i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)          # noqa: E731
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731
        self._psgd = {"P": P, "Q": Q, "p_ptrs": p_ptrs, "q_ptrs": q_ptrs, "p_mc": p_mc, "q_mc": q_mc, "pn": pn4, "qn": qn4,
                      "err": torch.zeros(fl.total, dtype=torch.float32, device=dev), "rank": r,
                      "tab": (i64([m[0] for m in mats]), i32([m[1] for m in mats]), i32([m[2] for m in mats]), i64(p_off), i64(q_off),
                              i64(rows), i64(blks), i64(elems)),
                      "counts": (rows[-1], blks[-1], elems[-1]), "ranges": [(lo, lo + m * n) for lo, m, n, _ in mats]}

    def _finish_powersgd(self):
        """After the backward pass: P = (G + E) Q for all matrices, mean over replicas, orthogonalise, Q = G^T P, mean, then
        G <- P Q^T and E <- G - P Q^T (``autodist/kernel/synchronization/compressor.py:208-284`` gives the algorithm); the
        optimizer kernels of the flights that hold matrices follow."""
        c = self._psgd
        if not c:
            return
        fl, E = self.flat, self.E
        compute = torch.cuda.current_stream()
        self._ready_event.record(compute)
        self.comm_stream.wait_event(self._ready_event)
        scale = 1.0 / self.world_size
        with torch.cuda.stream(self.comm_stream):
            rows, blks, elems = c["counts"]
            args = (fl.grad, c["err"], c["P"], c["Q"]) + c["tab"] + (c["rank"], rows, blks, elems)
            E.psgd_batched(0, *args)
            E.allreduce(*self.arena.ctx(), c["p_ptrs"], c["p_mc"], 0, c["pn"], None, None, None, scale, self._comm_blocks(c["pn"], bool(c["p_mc"])))
            E.psgd_batched(1, *args)
            E.psgd_batched(2, *args)
            E.allreduce(*self.arena.ctx(), c["q_ptrs"], c["q_mc"], 0, c["qn"], None, None, None, scale, self._comm_blocks(c["qn"], bool(c["q_mc"])))
            E.psgd_batched(3, *args)
            for lo, hi in self._psgd_flights:
                self._update_range(lo, hi)

    def _setup_ps_segments(self, flat_name):
        """Parameter-server parts as owned segments of the flat buffers (kernel ``reduce_scatter_update``)."""
        fl = self.flat
        self.ps_segments = []            # (start, length, owner) sorted by start; 4-element aligned
        self._ps_tables = {}
        by_var = {}
        for e in self.plan.ps_entries.values():
            by_var.setdefault(e.part.var_name, []).append(e)
        for var_name, entries in by_var.items():
            if var_name in self.sharded_rows:
                continue                              # kept as one shard per rank, outside the flat buffers' synchronisation
            name = flat_name[var_name]
            base, end = fl.offsets[name], fl.range_of([name])[1]
            p = fl.params[fl.names.index(name)]
            row = p.numel() // p.shape[0] if p.dim() > 0 and p.shape[0] > 0 else 1
            entries.sort(key=lambda e: e.part.offset)
            starts = [base + (e.part.offset * row if e.part.part_index is not None else 0) for e in entries]
            if any(st % 4 for st in starts):
                # shards of a tiny variable that do not start on 16-byte boundaries: the first owner takes all of it
                self.ps_segments.append((base, end - base, entries[0].owner))
                continue
            for i, e in enumerate(entries):
                stop = starts[i + 1] if i + 1 < len(entries) else end
                self.ps_segments.append((starts[i], stop - starts[i], e.owner))
        self.ps_segments.sort()
        if not self.ps_segments:
            return
        dev = self.device
        mine = [(st, ln) for st, ln, ow in self.ps_segments if ow == self.rank]
        self._state_offset = {}
        off = 0
        for st, ln in mine:
            self._state_offset[st] = off
            off += ln
        n = max(off, 4)
        self.ps_master = torch.zeros(n, dtype=torch.float32, device=dev)
        for st, ln in mine:
            o = self._state_offset[st]
            self.ps_master[o:o + ln].copy_(fl.master[st:st + ln])
        self.ps_s1 = torch.zeros(n, dtype=torch.float32, device=dev) if self._needs_slot1() else None
        if self.opt_kind == "Adagrad":
            self.ps_s1.fill_(float(self.opt_info.optimizer.param_groups[0].get("initial_accumulator_value", 0.0)))
        self.ps_s2 = torch.zeros(n, dtype=torch.float32, device=dev) if self.opt_kind in ("Adam", "AdamW") else None

    # ---- row-sparse variables sharded over all ranks: K4 (scatter-add to owners) / K5 (gather from owners) ----------
    def _row_shard_candidates(self):
        return row_shard_candidates(self.item, self.plan, not isinstance(self.module, _AutogradModel))

    def _setup_sharded_rows(self, row_sharded):
        if not row_sharded:
            return
        arena = self.arena if self.world_size > 1 else LocalArena(self.device)
        self._rows_arena = arena
        for var_name, p in row_sharded.items():
            full = p.data
            if self.world_size > 1:
                # rank 0's initial values, like every other variable
                full = full.to(self.device, torch.float32).contiguous()
                self.backend.broadcast_(full, 0)
            st = ShardedRows(self, var_name, p, full, arena)
            del full
            self.sharded_rows[var_name] = st
            p._sparse_rows = st                      # ops.functional.sparse_lookup and the fused models route through it

    def _finish_rows(self):
        """After the last push of a step: meet the peers (every rank's rows have landed), then every owner updates its shards."""
        if not self.sharded_rows:
            return
        if self.world_size > 1:
            self.E.sym_barrier(*self.arena.ctx(1), 1)
        for st in self.sharded_rows.values():
            st.update()

    def _apply_optimizer(self, p, gr, s1, s2, p16, group=0):
        g = self.opt_info.optimizer.param_groups[group]
        lr = self.lrs[group:group + 1]
        if self.opt_kind in ("Adam", "AdamW"):
            b1, b2 = g["betas"]
            self.E.adam_update(p, gr, s1, s2, p16, lr, b1, b2, g["eps"], g["weight_decay"], self.opt_kind == "AdamW", self.opt_step, 1.0)
        elif self.opt_kind == "SGD":
            self.E.sgd_update(p, gr, s1 if g.get("momentum", 0) != 0 else None, p16, lr, g["momentum"], g["dampening"], g["weight_decay"],
                              g["nesterov"], self.opt_step, 1.0)
        else:
            self.E.adagrad_update(p, gr, s1, p16, lr, g["eps"], g["weight_decay"], 1.0)

    def _ps_table(self, lo, hi):
        """Device tables of this rank's owned segments inside [lo, hi) (cached per flight)."""
        key = (lo, hi)
        if key not in self._ps_tables:
            inside = [(st, ln, ow) for st, ln, ow in self.ps_segments if st >= lo and st + ln <= hi]
            mine = [(st, ln) for st, ln, ow in inside if ow == self.rank]
            starts = [st for st, _ in mine] or [0]
            lens = [ln for _, ln in mine] or [0]
            state = [self._state_offset[st] for st, _ in mine] or [0]
            local = getattr(self, "_local_segments", set())
            flags = [1 if st in local else 0 for st, _ in mine] or [0]
            prefix = [0]
            for ln in lens:
                prefix.append(prefix[-1] + ln)
            t = lambda v: torch.tensor(v, dtype=torch.int64, device=self.device)   # noqa: E731
            total = sum(ln for _, ln, _ in inside)
            self._ps_tables[key] = (bool(inside), t(starts), t(lens), t(state), t(prefix), total, t(flags) if any(flags) else None)
        return self._ps_tables[key]

    def _ps_update_range(self, lo, hi):
        any_inside, starts, lens, state, prefix, total, flags = self._ps_table(lo, hi)
        if not any_inside:
            return 0
        g = self.opt_info.optimizer.param_groups[0]
        kind = {"SGD": 0, "Adam": 1, "AdamW": 1, "Adagrad": 2}[self.opt_kind]
        b1, b2 = g.get("betas", (0.0, 0.0))
        blocks = max(8, min(self.E.MAX_COMM_BLOCKS, total // (4 * 512 * self.world_size) + 1))
        use_mc = os.environ.get("AUTODIST_PS_MULTIMEM", "1") == "1"      # through the switch when the fabric offers multicast
        self.E.reduce_scatter_update(*self.arena.ctx(), self._grad_sym["ptrs"], self._p16_sym, self._p32_sym,
                                     self._grad_sym["mc"] if use_mc else 0, self._p16_mc if use_mc else 0, self._p32_mc if use_mc else 0,
                                     self.ps_master,
                                     self.ps_s1, self.ps_s2, starts, lens, state, flags, prefix, kind, self.lr, self.opt_step,
                                     b1, b2, g.get("eps", 1e-8), g.get("weight_decay", 0.0), g.get("momentum", 0.0), 1.0,
                                     self.opt_kind == "AdamW", bool(g.get("nesterov", False)), 1.0 / self.world_size, blocks)
        return 1

    def _policy_for(self, lo, hi):
        """Split [lo, hi) by the bucket policies that cover it."""
        out = []
        for blo, bhi, wd, ef, _ in self.range_wire:
            a, b = max(lo, blo), min(hi, bhi)
            if a < b:
                out.append((a, b, wd, ef))
        return out

    def _on_grad_ready(self, lo, hi):
        """Called by the model's backward pass when gradients [lo, hi) are final."""
        compute = torch.cuda.current_stream()
        self._ready_event.record(compute)
        self.comm_stream.wait_event(self._ready_event)
        keys = [f"g{gk}/i{ik}" for a, z, gk, ik in getattr(self, "_range_key", ()) if a < hi and z > lo]
        if self._flight_log is not None:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(self.comm_stream)
            try:
                self._launch_flight(lo, hi, keys)
            finally:
                t1.record(self.comm_stream)
                self._flight_log.append((lo, hi, t0, t1))
            return
        self._launch_flight(lo, hi, keys)

    def _launch_flight(self, lo, hi, keys):
        with nvtx.annotate(f"flight [{lo}, {hi}) {' '.join(keys[:4])}"), torch.cuda.stream(self.comm_stream):
            if getattr(self, "_relaxed", None):
                self._relaxed_push(lo, hi)               # this worker's gradient goes to the owners now; no collective, no local update
                self.launches_per_step += 1
                return
            if self.world_size > 1:
                for a, b, wd, ef in self._policy_for(lo, hi):
                    self._all_reduce_range(a, b, wd, ef)
                covered = self._policy_for(lo, hi)
                self.launches_per_step += self._ps_update_range(lo, hi)
            else:
                covered = [(lo, hi, None, False)]
            if (lo, hi) in getattr(self, "_deferred_ranges", ()):
                return                                   # clipped parameters inside: updated once the global norm is known
            if self._psgd and any(a < hi and z > lo for a, z in self._psgd["ranges"]):
                self._psgd_flights.append((lo, hi))      # holds matrices that travel as factors: updated after decompression
                return
            for a, b, _, _ in covered:
                self._update_range(a, b)
            self.launches_per_step += 2 * len(covered)

    def _comm_blocks(self, n_elems, nvls):
        """Blocks of one all-reduce launch: enough to fill the links, few enough to leave the SMs to the GEMMs that
        run next to it (the in-switch reduction needs far fewer threads than peer loads/stores)."""
        forced = int(os.environ.get("AUTODIST_COMM_BLOCKS", "0"))
        cap = forced or (64 if nvls else 96)
        return max(1, min(cap, n_elems // (4 * 512 * self.world_size) + 1))

    def _all_reduce_range(self, lo, hi, wd, ef):
        n = hi - lo
        scale = 1.0 / self.world_size
        ctx = self.arena.ctx()
        if wd is None:
            ptrs = self._grad_sym["ptrs"] + lo * 4
            mc = self._grad_sym["mc"] + lo * 4 if self._grad_sym["mc"] else 0
            self.E.allreduce(*ctx, ptrs, mc, 0, n, None, None, None, scale, self._comm_blocks(n, bool(mc)))
        else:
            ptrs = self._wire_ptrs + lo * 2
            mc = self._wire_mc + lo * 2 if self._wire_mc else 0
            g = self.flat.grad[lo:hi]
            self.E.allreduce(*ctx, ptrs, mc, WIRE[wd], n, g, self._residual[lo:hi] if ef else None, g, scale,
                             self._comm_blocks(n, bool(mc)))

    # ------------------------------------------------------------------ step
    def _run_model(self, train_op, nodes, feeds):
        all_nodes = list(nodes)
        if train_op.loss_node not in all_nodes:
            all_nodes.append(train_op.loss_node)
        self.E.increment(self.opt_step)
        self.launches_per_step = 0
        self._rows_sync_pending, self._rows_dirty = True, False
        self._psgd_flights = []
        if self._flight_log is not None:
            self._flight_log.clear()
            self._step_start = torch.cuda.Event(enable_timing=True)
            self._step_start.record()
        values = self.forward(all_nodes, feeds, grad=True)
        self._finish_rows()
        self._finish_powersgd()
        self._finish_relaxed()
        # the optimizer kernels of the last flights run on the communication stream: join it
        self._done_event.record(self.comm_stream)
        torch.cuda.current_stream().wait_event(self._done_event)
        return values

    def flight_report(self):
        """Flights of the last step, in launch order: ``(lo, hi, start_ms, ms)`` with the start measured from the first
        kernel of the step and ``ms`` the time the flight's kernels (collective + optimizer) held the communication
        stream. Needs ``AUTODIST_FLIGHT_TIMING=1``; synchronises the device."""
        if not self._flight_log or self._step_start is None:
            return []
        torch.cuda.synchronize(self.device)
        return [(lo, hi, self._step_start.elapsed_time(t0), t0.elapsed_time(t1)) for lo, hi, t0, t1 in self._flight_log]

    def train_step(self, train_op, nodes, feeds):
        self._sync_lr()
        if not self._use_graph or self._flight_log is not None:
            values = self._run_model(train_op, nodes, feeds)
        else:
            values = self._graphed_step(train_op, nodes, feeds)
        self.global_step += 1
        if self.global_step % 50 == 1:
            self.check_errors()
        return [v.detach() if isinstance(v, torch.Tensor) else v for v in values[:len(nodes)]]

    def _graphed_step(self, train_op, nodes, feeds):
        if any(n is not train_op.loss_node for n in nodes):
            return self._run_model(train_op, nodes, feeds)       # fetches beyond the loss: run eagerly
        # one capture serves both `run(train_op)` and `run([loss, train_op])`: the loss is always computed
        requested, nodes = len(nodes), [train_op.loss_node]
        key = (id(train_op), tuple((k, tuple(v.shape)) for k, v in sorted(feeds.items())))
        if self._graph is not None and self._graph[0] != key:
            self._graph = None
        if self._graph is None:
            if self._warm_steps < 2:
                # run eagerly first: lazy initialisation (workspaces, kernel attributes) must not happen during capture
                self._warm_steps += 1
                return self._run_model(train_op, nodes, feeds)[:requested]
            static = {k: v.clone() for k, v in feeds.items()}
            torch.cuda.synchronize()
            if self.world_size > 1:
                dist.barrier(group=self.backend.group)
            graph = torch.cuda.CUDAGraph()
            from autodist_b200 import ops
            before = ops.launch_count
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    out = self._run_model(train_op, nodes, static)
            except Exception as e:       # a program that cannot be captured keeps running eagerly
                logging.warning("CUDA graph capture failed (%s); continuing with eager launches", e)
                self._use_graph = False
                torch.cuda.synchronize()
                return self._run_model(train_op, nodes, feeds)[:requested]
            self.graph_kernels = ops.launch_count - before   # kernels of this extension per replay
            self._graph = (key, graph, static, out)
            torch.cuda.synchronize()
            if self.world_size > 1:
                dist.barrier(group=self.backend.group)
            # the capture itself does not execute: fall through to a replay for this step
        _, graph, static, out = self._graph
        for k, v in feeds.items():
            static[k].copy_(v, non_blocking=True)
        graph.replay()
        return out[:requested]

    def sync_and_update(self, train_op):
        return

    def check_errors(self):
        self.module.check_error()
        if self.arena is not None:
            self.arena.check()
        elif getattr(self, "_rows_arena", None) is not None:
            self._rows_arena.check()

    def before_read(self):
        return

    # ------------------------------------------------------------------ state
    def variable_value(self, name):
        st = self.sharded_rows.get(name)
        if st is not None:
            return st.gather(st.master)
        return self._params[name].detach()

    def optimizer_slots(self):
        names = {"Adam": ("exp_avg", "exp_avg_sq"), "AdamW": ("exp_avg", "exp_avg_sq"), "SGD": ("momentum_buffer",),
                 "Adagrad": ("sum",)}[self.opt_kind]
        out = {}
        bufs = [self.slot1, self.slot2]
        if self.ps_segments:
            # slots of parameter-server segments live with their owners: gather them into full-size buffers
            merged = []
            for local, owned in zip(bufs, (self.ps_s1, self.ps_s2)):
                if local is None:
                    merged.append(None)
                    continue
                full_buf = local.clone()
                for st, ln, ow in self.ps_segments:
                    full_buf[st:st + ln].zero_()
                    if ow == self.rank:
                        o = self._state_offset[st]
                        full_buf[st:st + ln].copy_(owned[o:o + ln])
                mask = torch.zeros_like(full_buf)
                for st, ln, ow in self.ps_segments:
                    mask[st:st + ln] = 1
                part = full_buf * mask
                dist.all_reduce(part, group=self.backend.group)
                merged.append(torch.where(mask.bool(), part, full_buf))
            bufs = merged
        for name, p in zip(self.flat.names, self.flat.params):
            full = self.item.name_of_parameter(p)[:-2]
            o, n = self.flat.offsets[name], p.numel()
            for slot, buf in zip(names, bufs):
                if buf is not None:
                    out[f"{full}/{slot}"] = buf[o:o + n].view(p.shape).clone()
            out[f"{full}/step"] = torch.as_tensor(float(self.global_step))
        for st in self.sharded_rows.values():
            full = st.var[:-2]
            for slot, buf in zip(names, (st.s1, st.s2)):
                if buf is not None:
                    out[f"{full}/{slot}"] = st.gather(buf)
            out[f"{full}/step"] = torch.as_tensor(float(self.global_step))
        return out

    def load_optimizer_slots(self, slots, default_step=0):
        names = {"Adam": ("exp_avg", "exp_avg_sq"), "AdamW": ("exp_avg", "exp_avg_sq"), "SGD": ("momentum_buffer",),
                 "Adagrad": ("sum",)}[self.opt_kind]
        for name, p in zip(self.flat.names, self.flat.params):
            full = self.item.name_of_parameter(p)[:-2]
            o, n = self.flat.offsets[name], p.numel()
            for slot, buf in zip(names, (self.slot1, self.slot2)):
                key = f"{full}/{slot}"
                if buf is not None and key in slots:
                    buf[o:o + n].copy_(slots[key].reshape(-1).to(self.device))
        # Slots of parameter-server segments live with their owners, slots of a row-sharded table with the owner of each
        # row block: copy this rank's parts out of the full-size buffers just filled.
        for st_, ln, ow in getattr(self, "ps_segments", []):
            if ow == self.rank:
                o = self._state_offset[st_]
                for owned, full_buf in ((self.ps_s1, self.slot1), (self.ps_s2, self.slot2)):
                    if owned is not None and full_buf is not None:
                        owned[o:o + ln].copy_(full_buf[st_:st_ + ln])
        for st in self.sharded_rows.values():
            full = st.var[:-2]
            loaded = [slots.get(f"{full}/{slot}") for slot in names] + [None]
            st.load_slots(loaded[0], loaded[1] if len(names) > 1 else None)
        self.opt_step.fill_(int(default_step))

    def after_restore(self):
        self.flat.refresh_bf16()
        self.opt_step.fill_(self.global_step)
        for st in self.sharded_rows.values():
            st.load(st.param.data)                   # the restore wrote the full table into the parameter
        for st_, ln, ow in getattr(self, "ps_segments", []):
            if ow == self.rank:
                o = self._state_offset[st_]
                self.ps_master[o:o + ln].copy_(self.flat.master[st_:st_ + ln])

    def close(self):
        r = getattr(self, "_relaxed", None)
        if r:
            # leaving: publish a step no peer can be ahead of, so that nobody waits for a worker that has finished
            torch.cuda.synchronize()
            self.E.staleness_gate(*self.arena.ctx(), r["cptrs"], 1 << 30, -1, None, None)
            torch.cuda.synchronize()
            self._relaxed = None


class _AutogradModel:
    """Adapter that gives an ordinary autograd program the flat-buffer face the fused engine expects."""

    def __init__(self, graph_item):
        self.item = graph_item
        self.flat = None
        self.grad_ready = None

    def materialize(self, device, grad_alloc=None, master_alloc=None, p16_alloc=None, exclude=()):
        """``exclude``: ids of parameters that stay outside the flat buffers (row-sharded tables: their full value stays
        where it is, on the host, as the source for shards and checkpoints)."""
        from autodist_b200.ops.flat import FlatParams
        with torch.no_grad():
            for b in self.item.root.buffers():
                b.data = b.data.to(device)
        named = [(n[:-2], p) for n, p in self.item.named_parameters() if id(p) not in exclude]
        frozen = [p for _, p in named if not p.requires_grad]
        with torch.no_grad():
            for p in frozen:
                p.data = p.data.to(device)
        self.flat = FlatParams([(n, p) for n, p in named if p.requires_grad], device, grad_alloc,
                               master_alloc=master_alloc, p16_alloc=p16_alloc)
        for n, p in zip(self.flat.names, self.flat.params):
            p._bf16_view = self.flat.w16[n]          # the optimizer kernels keep this compute copy current: no per-call cast
        return self.flat

    def check_error(self):
        from autodist_b200.ops.functional import check_errors
        check_errors()


class FlatAutogradEngine(FusedStepEngine):
    """Any ``torch.autograd`` program on the fused communication path.

    Parameters and gradients are re-homed into flat buffers (gradients in symmetric memory); autograd accumulates
    into those views in place, post-accumulate hooks report finished parameters, and as soon as a *flight* (a run
    of consecutive parameters, at least ``AUTODIST_FLIGHT_MB`` of gradients) is complete its all-reduce /
    reduce-scatter kernel and the fused optimizer kernel run on the communication stream while autograd continues.
    This is how the CNN benchmarks and LM1B (autograd programs over the hand-written kernels) use the same synchronisation
    kernels as the hand-scheduled models.
    """

    @staticmethod
    def supports_autograd(graph_item, plan):
        if len(graph_item.optimizers) != 1:
            return False
        params = [p for _, p in graph_item.named_parameters() if p.requires_grad]
        if not params or any(p.dtype != torch.float32 for p in params):
            return False
        updated = graph_item.updated_variable_names()
        if any(graph_item.name_of_parameter(p) not in updated for p in params):
            return False
        # Row-sparse variables: tables that can live as one row shard per rank, or vectors (whose gradient arrives dense).
        # Any other sparse variable keeps the generic engine's row exchange.
        sharded = row_shard_candidates(graph_item, plan, False)
        for name, p in graph_item.named_parameters():
            var = graph_item.variables.get(name)
            if var is not None and var.sparse_grad and p.requires_grad and name not in sharded and p.dim() != 1:
                return False
        # Global-norm clipping needs the complete reduced gradient before any update: possible for variables whose
        # gradients are all-reduced (every replica then applies the same clipped update), not for parameter-server parts,
        # whose kernel reduces and updates in one pass.
        ps_vars = {e.part.var_name for e in plan.ps_entries.values()}
        for op in graph_item.train_ops:
            if op.clip_global_norm and plan.replica.world_size > 1:
                if any(graph_item.name_of_parameter(p) in ps_vars for p in op.clip_global_norm[1]):
                    return False
        if len([op for op in graph_item.train_ops if op.clip_global_norm]) > 1:
            return False
        return FusedStepEngine.supports(graph_item, plan, None)

    def __init__(self, graph_item, plan, backend, device):
        super().__init__(graph_item, plan, backend, device, _AutogradModel(graph_item))
        # The whole step of an autograd program (forward, backward, hooks and their flights) is captured into one CUDA
        # graph after two eager steps; AUTODIST_AUTOGRAD_GRAPH=0 keeps eager launches (needed for programs whose
        # control flow depends on data). A capture that fails falls back to eager launches by itself.
        self._use_graph = os.environ.get("AUTODIST_AUTOGRAD_GRAPH", "1") == "1"
        self._warm_needed = 3
        fl = self.flat
        limit = int(float(os.environ.get("AUTODIST_FLIGHT_MB", "32")) * (1 << 20) / 4)
        # flights in backward order: consecutive parameters from the end of the flat buffer
        self._flight_of, self._flights = {}, []
        hi = fl.total
        names = list(fl.names)
        members = []
        for name in reversed(names):
            members.append(name)
            lo = fl.offsets[name]
            if hi - lo >= limit or name == names[0]:
                self._flights.append({"lo": lo, "hi": hi, "need": len(members), "have": 0, "sent": False, "seen": set()})
                for m in members:
                    self._flight_of[m] = len(self._flights) - 1
                members, hi = [], lo
        self._setup_clip()
        self._setup_gathered_weights()
        for name, p in zip(fl.names, fl.params):
            hook = self._make_hook(name)
            p.register_post_accumulate_grad_hook(hook)
            # kernels that add a gradient straight into the flat buffer (weight-gradient GEMMs, batch-norm parameter sums)
            # bypass autograd's accumulation and report completion through this attribute instead
            p._direct_grad = os.environ.get("AUTODIST_DIRECT_GRAD", "1") == "1"
            p._grad_ready_hook = hook

    def _setup_gathered_weights(self):
        """All-gather fused into the consumer (K3): a large fully connected weight that the plan splits along axis 0 into one
        shard per rank (rank ``i`` owns block ``i``) is not written back to the other replicas after its owner's update.
        Its consumers - ``ops.functional.linear`` forward and input gradient - fetch the shards from their owners tile by
        tile inside the GEMM (``gemm_gathered_b`` / ``gemm_gathered_bt``, plain TMA loads over NVLink), so the weight crosses
        the links as bf16 tiles that are used at once instead of as fp32 + bf16 copies that are stored first. The reference
        reads such a variable from its parameter server, or from a mirror refreshed after every update
        (``autodist/kernel/synchronization/ps_synchronizer.py:175-176``, ``autodist/kernel/common/proxy_variable.py:96-114``)."""
        self.gathered_vars = {}
        self._local_segments = set()
        if self.world_size <= 1 or not self.ps_segments or os.environ.get("AUTODIST_GATHER_WEIGHTS", "1") != "1":
            return
        from autodist_b200.ops.functional import Linear
        min_bytes = float(os.environ.get("AUTODIST_GATHER_MIN_MB", "64")) * (1 << 20)
        fl, world = self.flat, self.world_size
        flat_of = {id(p): n for n, p in zip(fl.names, fl.params)}
        by_var = {}
        for e in self.plan.ps_entries.values():
            by_var.setdefault(e.part.var_name, []).append(e)
        seg_owner = {st: (ln, ow) for st, ln, ow in self.ps_segments}
        bases = [int(x) for x in self._p16_sym.tolist()]
        for m in self.item.root.modules():
            if not isinstance(m, Linear) or id(m.weight) not in flat_of:
                continue
            p = m.weight
            n_out, k_in = p.shape
            var_name = self.item.name_of_parameter(p)
            entries = sorted(by_var.get(var_name, []), key=lambda e: e.part.offset)
            rows = n_out // world
            if p.numel() * 2 < min_bytes or len(entries) != world or n_out % world or rows % 64 or k_in % 8:
                continue
            owners = [e.owner for e in entries]
            if sorted(owners) != list(range(world)) or any(e.part.axis != 0 or e.part.size != rows for e in entries):
                continue              # (every rank owns exactly one block, in any order)
            base = fl.offsets[flat_of[id(p)]]
            starts = [base + i * rows * k_in for i in range(world)]
            if any(seg_owner.get(st) != (rows * k_in, owners[i]) for i, st in enumerate(starts)):
                continue
            self._local_segments.update(starts)
            p._gathered = {"ptrs": [bases[owners[i]] + 2 * starts[i] for i in range(world)], "rows": rows}
            self.gathered_vars[var_name] = (flat_of[id(p)], rows, k_in, owners)
        if self.gathered_vars:
            logging.info("weights gathered inside their GEMMs instead of written back: %s", ", ".join(self.gathered_vars))

    def _refresh_gathered(self):
        """Bring every replica's copies of the gathered weights up to date (variable fetches, checkpoints): each owner
        contributes its rows."""
        fl = self.flat
        for name, rows, k_in, owners in self.gathered_vars.values():
            base = fl.offsets[name]
            n = rows * k_in
            blk = owners.index(self.rank)                      # the block this rank owns and keeps current
            mine = fl.master[base + blk * n: base + (blk + 1) * n].contiguous()
            parts = [torch.empty_like(mine) for _ in range(self.world_size)]
            dist.all_gather(parts, mine, group=self.backend.group)
            for i in range(self.world_size):
                t = parts[owners[i]]
                fl.master[base + i * n: base + (i + 1) * n].copy_(t)
                fl.p16[base + i * n: base + (i + 1) * n].copy_(t)

    def variable_value(self, name):
        if getattr(self, "gathered_vars", None) and name in self.gathered_vars:
            self._refresh_gathered()
        return super().variable_value(name)

    def _setup_clip(self):
        """Global-norm clipping (``minimize(..., clip_global_norm=(max_norm, parameters))``): flights that carry a clipped
        parameter are reduced as they complete, but their optimizer kernels wait until the norm of all clipped gradients is
        known (``sumsq`` over the reduced ranges into a device scalar, ``clip_scale`` in place) - the norm never visits the host."""
        self._clip = None
        ops_ = [op for op in self.item.train_ops if op.clip_global_norm]
        if not ops_:
            return
        max_norm, params = ops_[0].clip_global_norm
        fl = self.flat
        flat_of = {id(p): n for n, p in zip(fl.names, fl.params)}
        ranges = sorted((fl.offsets[flat_of[id(p)]], fl.offsets[flat_of[id(p)]] + p.numel()) for p in params if id(p) in flat_of)
        deferred = []
        for i, f in enumerate(self._flights):
            if any(lo < f["hi"] and hi > f["lo"] for lo, hi in ranges):
                deferred.append(i)
                f["deferred"] = True
        self._clip = {"max_norm": float(max_norm), "ranges": ranges, "flights": deferred,
                      "acc": torch.zeros(1, dtype=torch.float32, device=self.device)}
        self._deferred_ranges = {(self._flights[i]["lo"], self._flights[i]["hi"]) for i in deferred}

    def _finish_clipped(self):
        c = getattr(self, "_clip", None)
        if not c:
            return
        fl = self.flat
        compute = torch.cuda.current_stream()
        self._ready_event.record(compute)
        self.comm_stream.wait_event(self._ready_event)
        with torch.cuda.stream(self.comm_stream):          # behind the reductions of every flight
            c["acc"].zero_()
            for lo, hi in c["ranges"]:
                self.E.sumsq(fl.grad[lo:hi], c["acc"], 1.0)
            for lo, hi in c["ranges"]:
                self.E.clip_scale(fl.grad[lo:hi], c["acc"], c["max_norm"])
            for i in c["flights"]:
                f = self._flights[i]
                for a, b, _, _ in (self._policy_for(f["lo"], f["hi"]) if self.world_size > 1 else [(f["lo"], f["hi"], None, False)]):
                    self._update_range(a, b)

    def _make_hook(self, name):
        def hook(param):
            f = self._flights[self._flight_of[name]]
            if name in f["seen"]:
                return          # a directly accumulated gradient may be reported by its kernel's wrapper and by autograd
            f["seen"].add(name)
            f["have"] += 1
            if f["have"] == f["need"] and not f["sent"]:
                f["sent"] = True
                self._on_grad_ready(f["lo"], f["hi"])
        return hook

    def _run_model(self, train_op, nodes, feeds):
        all_nodes = list(nodes)
        if train_op.loss_node not in all_nodes:
            all_nodes.append(train_op.loss_node)
        self.E.increment(self.opt_step)
        self.launches_per_step = 0
        self._rows_sync_pending, self._rows_dirty = True, False
        self._psgd_flights = []
        if self._flight_log is not None:
            self._flight_log.clear()
            self._step_start = torch.cuda.Event(enable_timing=True)
            self._step_start.record()
        fl = self.flat
        fl.grad.zero_()
        for f in self._flights:
            f["have"], f["sent"] = 0, False
            f["seen"].clear()
        for name, p in zip(fl.names, fl.params):
            p.grad = fl.g[name]                      # autograd adds into the flat views in place
            p._pending_uses = 0
        values = self.forward(all_nodes, feeds, grad=True)
        values[all_nodes.index(train_op.loss_node)].backward()
        for f in self._flights:                      # parameters that received no gradient this step: still synchronised
            if not f["sent"]:
                f["sent"] = True
                self._on_grad_ready(f["lo"], f["hi"])
        self._finish_rows()
        self._finish_clipped()
        self._finish_powersgd()
        self._finish_relaxed()
        self._done_event.record(self.comm_stream)
        torch.cuda.current_stream().wait_event(self._done_event)
        return values
