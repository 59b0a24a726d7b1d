"""Feed / fetch remapping between the user's single-device view and this rank's replica.

Capability parity with ``autodist/remapper.py:29-313``:

* **feed** - a value fed to a placeholder with a polymorphic (``None``) dimension
  is split along that dimension between the replicas of this node with
  ``numpy.array_split`` semantics (uneven allowed); this process keeps the chunk
  of its own replica. Placeholders without such a dimension get the same value
  on every replica.
* **fetch** - a ``train_op`` runs on every replica and yields ``None``; a tensor
  that carries the batch dimension is concatenated over the node's replicas;
  anything else is replica 0's value (``AUTODIST_FETCH_MODE=local`` returns this
  replica's own value without communication); a variable yields its full
  (merged) value.
"""
import numpy as np
import torch
import torch.fx as fx
from torch import nn

from autodist_b200.const import ENV
from autodist_b200.graph_item import TrainOp


class PinnedStager:
    """Pinned staging buffers for host values that are not pinned themselves, ``depth`` per placeholder, used in rotation.

    ``upload`` copies the value into the next buffer on the host and starts an asynchronous host-to-device copy from it.
    Each buffer remembers the event recorded after its last copy; before the host writes into a buffer again it waits for
    that event, so a step whose copy is still queued behind earlier work (a replayed CUDA graph returns at once) never
    reads a batch that the host has already overwritten."""

    def __init__(self, device, depth=2):
        self.device = torch.device(device)
        self.depth = depth
        self._slots = {}          # name -> {"bufs": [...], "events": [...], "next": int}

    def upload(self, name, t):
        slot = self._slots.get(name)
        if slot is None or slot["bufs"][0].shape != t.shape or slot["bufs"][0].dtype != t.dtype:
            slot = {"bufs": [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for _ in range(self.depth)],
                    "events": [None] * self.depth, "next": 0}
            self._slots[name] = slot
        i = slot["next"]
        slot["next"] = (i + 1) % self.depth
        if slot["events"][i] is not None:
            slot["events"][i].synchronize()          # the copy that last read this buffer has finished
        slot["bufs"][i].copy_(t)
        out = slot["bufs"][i].to(self.device, non_blocking=True)
        ev = slot["events"][i] or torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        slot["events"][i] = ev
        return out


def _chunk_bounds(n, k, i):
    q, r = divmod(n, k)
    start = i * q + min(i, r)
    return start, start + q + (1 if i < r else 0)


class Remapper:
    def __init__(self, graph_item, plan, device, local_group=None):
        self._item = graph_item
        self._plan = plan
        self._device = torch.device(device)
        self._local_group = local_group
        self._num_local = plan.replica.num_local_replicas
        self._local_index = plan.replica.local_replica_index
        self._stager = PinnedStager(self._device) if self._device.type == "cuda" else None
        self.fetch_mode = ENV.AUTODIST_FETCH_MODE.val
        if plan.gate_mode != "sync":
            self.fetch_mode = "local"   # relaxed modes must not add a lock-step collective
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._last_chunk = {}
        self._prefetched = {}          # id(fed value) -> (value, placeholder name, device tensor, copy event, batch chunk)
        self._copy_stream = None

    # ------------------------------------------------------------------ feeds
    @property
    def num_local_replicas(self):
        """Replicas that this process feeds: a fed batch is split between them along its batch dimension."""
        return self._num_local

    def _to_device(self, name, value):
        if isinstance(value, torch.Tensor):
            t = value
        else:
            t = torch.from_numpy(np.ascontiguousarray(value))
        if self._device.type == "cpu":
            return t
        if t.device.type == "cpu":
            self.h2d_bytes += t.numel() * t.element_size()
            if not t.is_pinned():
                return self._stager.upload(name, t)
            return t.to(self._device, non_blocking=True)
        return t.to(self._device)

    def _remap_one(self, key, value):
        """One fed value -> (placeholder name, this replica's slice on the device in the placeholder's dtype)."""
        info = self._item.placeholder_of(key)
        if not isinstance(value, (torch.Tensor, np.ndarray)):
            value = np.asarray(value)
        if isinstance(value, np.ndarray) and value.dtype == np.float64 and info.dtype == torch.float32:
            value = value.astype(np.float32)
        dim = info.batch_dim
        if dim is not None and self._num_local > 1:
            lo, hi = _chunk_bounds(value.shape[dim], self._num_local, self._local_index)
            index = [slice(None)] * value.ndim
            index[dim] = slice(lo, hi)
            value = value[tuple(index)]
        if dim is not None:
            self._last_chunk[info.name] = value.shape[dim]
        t = self._to_device(info.name, value)
        if t.dtype != info.dtype and t.is_floating_point() and info.dtype.is_floating_point:
            t = t.to(info.dtype)
        return info.name, t

    def remap_feed(self, feed_dict):
        feeds = {}
        for key, value in (feed_dict or {}).items():
            staged = self._prefetched.pop(id(value), None)
            if staged is not None and staged[0] is value:
                # uploaded by `prefetch` while the previous step ran: the step only waits for that copy
                name, t, ev, chunk = staged[1], staged[2], staged[3], staged[4]
                torch.cuda.current_stream(self._device).wait_event(ev)
                t.record_stream(torch.cuda.current_stream(self._device))
                if chunk is not None:
                    self._last_chunk[name] = chunk
                feeds[name] = t
                continue
            name, t = self._remap_one(key, value)
            feeds[name] = t
        self._prefetched.clear()
        return feeds

    def prefetch(self, feed_dict):
        """Starts the upload of a later step's feed on a copy stream of its own, so that it overlaps the step that is
        running; ``remap_feed`` recognises the same value objects when they are fed and skips their copy. Values that
        are not fed next are simply dropped."""
        self._prefetched.clear()
        if self._device.type != "cuda" or not feed_dict:
            return
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self._device)
        current = dict(self._last_chunk)           # the running step's fetches are still cut with its own batch sizes
        with torch.cuda.stream(self._copy_stream):
            for key, value in feed_dict.items():
                name, t = self._remap_one(key, value)
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
                self._prefetched[id(value)] = (value, name, t, ev, self._last_chunk.get(name))
        self._last_chunk = current

    # ------------------------------------------------------------------ fetches
    def flatten_fetches(self, fetches):
        """Returns (leaves, rebuild) where rebuild(list of values) restores the fetch structure."""
        leaves = []

        def walk(obj):
            if isinstance(obj, (list, tuple)):
                subs = [walk(o) for o in obj]
                return lambda vals, subs=subs, kind=type(obj): kind(s(vals) for s in subs)
            if isinstance(obj, dict):
                subs = {k: walk(v) for k, v in obj.items()}
                return lambda vals, subs=subs: {k: s(vals) for k, s in subs.items()}
            leaves.append(obj)
            idx = len(leaves) - 1
            return lambda vals, idx=idx: vals[idx]

        rebuild = walk(fetches)
        return leaves, rebuild

    def classify(self, leaf):
        if isinstance(leaf, TrainOp):
            return "train_op"
        if isinstance(leaf, fx.Proxy):
            return "tensor"
        if isinstance(leaf, nn.Parameter):
            return "variable"
        if isinstance(leaf, str):
            name = leaf if leaf.endswith(":0") else leaf + ":0"
            if name in self._item.variables:
                return "variable"
            for n in self._item.tracer.graph.nodes:
                if n.name == leaf or n.name + ":0" == leaf:
                    return "tensor"
        raise TypeError(f"cannot fetch {leaf!r}")

    def node_of(self, leaf):
        if isinstance(leaf, fx.Proxy):
            return leaf.node
        for n in self._item.tracer.graph.nodes:
            if n.name == leaf or n.name + ":0" == leaf:
                return n
        raise KeyError(leaf)

    def _is_batch_tensor(self, value):
        if not isinstance(value, torch.Tensor) or value.dim() == 0 or not self._last_chunk:
            return False
        return value.shape[0] in set(self._last_chunk.values())

    def remap_fetch(self, value, to_numpy=True):
        """Merge one fetched tensor over the node's replicas and bring it to the host."""
        if not isinstance(value, torch.Tensor):
            return value
        if self._num_local > 1 and self.fetch_mode != "local":
            import torch.distributed as dist
            if self._is_batch_tensor(value):
                counts = [torch.zeros(1, dtype=torch.int64, device=value.device) for _ in range(self._num_local)]
                dist.all_gather(counts, torch.tensor([value.shape[0]], dtype=torch.int64, device=value.device),
                                group=self._local_group)
                counts = [int(c.item()) for c in counts]
                cap = max(counts)
                pad = value.new_zeros((cap,) + tuple(value.shape[1:]))
                pad[:value.shape[0]] = value
                out = [torch.empty_like(pad) for _ in range(self._num_local)]
                dist.all_gather(out, pad, group=self._local_group)
                value = torch.cat([o[:c] for o, c in zip(out, counts)])
            else:
                value = value.contiguous().clone()
                dist.broadcast(value, src=self._plan.replica.local_ranks[0], group=self._local_group)
        if value.device.type != "cpu":
            self.d2h_bytes += value.numel() * value.element_size()
        if not to_numpy:
            return value.cpu()
        host = value.detach().cpu()
        if host.dtype == torch.bfloat16:
            host = host.float()
        return np.array(host.numpy(), copy=True) if value.device.type == "cpu" else host.numpy()
