"""Communication backends behind the synchronizers.

``TorchDistBackend`` drives ``torch.distributed`` (gloo between CPU ranks, NCCL
between GPUs). It is the plumbing for CPU runs and, on GPUs, the *baseline* the
fused symmetric-memory kernels of ``fused_comm.py`` are measured against. The
reference has no counterpart module: its collectives are TensorFlow ops
(``autodist/kernel/synchronization/compressor.py:84-96``).
"""
import torch
import torch.distributed as dist


class LocalBackend:
    """World of one replica: every collective is the identity."""
    rank = 0
    world_size = 1
    name = "local"

    def compressed_all_reduce_mean_(self, flat, wire_dtype, residual):
        if wire_dtype is not None:
            t = flat + residual if residual is not None else flat
            c = t.to(wire_dtype).to(flat.dtype)
            if residual is not None:
                residual.copy_(t - c)
            flat.copy_(c)
        return flat

    def reduce_mean_to_(self, flat, owner):
        return flat

    def broadcast_(self, tensor, src):
        return tensor

    def all_gather_rows(self, indices, values):
        return indices, values

    def all_reduce_sum_(self, tensor):
        return tensor

    def all_gather_counts(self, n):
        return [n]

    def barrier(self):
        return

    def all_reduce_scalar(self, value, op="sum"):
        return value


class TorchDistBackend(LocalBackend):
    name = "torch.distributed"

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.bytes_reduced = 0

    def compressed_all_reduce_mean_(self, flat, wire_dtype, residual):
        self.bytes_reduced += flat.numel() * (flat.element_size() if wire_dtype is None else 2)
        if wire_dtype is None:
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world_size)
            return flat
        t = flat.add(residual) if residual is not None else flat
        c = t.to(wire_dtype)
        if residual is not None:
            torch.sub(t, c.to(flat.dtype), out=residual)
        # Pre-divide so that the 16-bit sum cannot overflow.
        c.div_(self.world_size)
        if c.device.type == "cpu" and wire_dtype is torch.float16:
            # gloo has no fp16 sum on every build: widen on the wire for CPU plumbing runs.
            w = c.float()
            dist.all_reduce(w, group=self.group)
            flat.copy_(w.to(wire_dtype))
        else:
            dist.all_reduce(c, group=self.group)
            flat.copy_(c)
        return flat

    def reduce_mean_to_(self, flat, owner):
        dist.reduce(flat, dst=owner, group=self.group)
        if self.rank == owner:
            flat.div_(self.world_size)
        return flat

    def broadcast_(self, tensor, src):
        dist.broadcast(tensor, src=src, group=self.group)
        return tensor

    def all_reduce_sum_(self, tensor):
        self.bytes_reduced += tensor.numel() * tensor.element_size()
        dist.all_reduce(tensor, group=self.group)
        return tensor

    def all_gather_counts(self, n, device="cpu"):
        mine = torch.tensor([n], dtype=torch.int64, device=device)
        out = [torch.zeros_like(mine) for _ in range(self.world_size)]
        dist.all_gather(out, mine, group=self.group)
        return [int(t.item()) for t in out]

    def all_gather_rows(self, indices, values):
        """Concatenate every rank's (indices, values); ranks may contribute different row counts."""
        counts = self.all_gather_counts(indices.numel(), indices.device)
        cap = max(counts) if counts else 0
        if cap == 0:
            return indices, values
        pad_i = indices.new_zeros(cap)
        pad_i[:indices.numel()] = indices
        pad_v = values.new_zeros((cap,) + tuple(values.shape[1:]))
        pad_v[:values.shape[0]] = values
        gi = [torch.empty_like(pad_i) for _ in range(self.world_size)]
        gv = [torch.empty_like(pad_v) for _ in range(self.world_size)]
        dist.all_gather(gi, pad_i, group=self.group)
        dist.all_gather(gv, pad_v, group=self.group)
        return (torch.cat([g[:c] for g, c in zip(gi, counts)]),
                torch.cat([g[:c] for g, c in zip(gv, counts)]))

    def barrier(self):
        dist.barrier(group=self.group)

    def all_reduce_scalar(self, value, op="sum"):
        t = torch.tensor([float(value)], dtype=torch.float64)
        if dist.get_backend(self.group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX,
                               "min": dist.ReduceOp.MIN}[op], group=self.group)
        return float(t.item())
