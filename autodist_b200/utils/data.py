"""Record files and the background batch feeder.

A record file holds fixed-size records, the fields of one sample back to back (``write_records``). ``RecordFeeder``
iterates over it in batches: native worker threads (``csrc/host/batch_feeder.cpp``) gather the (shuffled) records of the
next batches into a ring of pinned host buffers while the training loop consumes the current one, so the loop never waits
for the host and ``Session.run(..., prefetch=next_batch)`` can start the upload of the next batch while a step runs.

The reference's benchmark drivers read TFRecord files through ``tf.data`` pipelines
(``examples/benchmark/utils/input_pipeline.py:82-131``, ``imagenet_preprocessing.py:242-316``: interleave, shuffle, batch,
prefetch); this is the same role for pre-processed fixed-size samples.
"""
import json
import os

import numpy as np
import torch

_NP = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64, torch.int32: np.int32, torch.uint8: np.uint8,
       torch.int8: np.int8, torch.float64: np.float64, torch.bool: np.bool_}


def _fields_layout(fields):
    layout, off = [], 0
    for name, (shape, dtype) in fields.items():
        nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        layout.append((name, tuple(shape), dtype, off, nbytes))
        off += nbytes
    return layout, off


def write_records(path, arrays):
    """Writes ``arrays`` (name -> array / tensor ``[N, ...]``, in this order) as ``N`` fixed-size records and a ``.json``
    side file describing the fields. Returns the ``fields`` mapping to give to ``RecordFeeder``."""
    tensors = {k: (v if isinstance(v, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(v))).contiguous() for k, v in arrays.items()}
    n = {int(t.shape[0]) for t in tensors.values()}
    if len(n) != 1:
        raise ValueError("all arrays need the same first dimension")
    n = n.pop()
    fields = {k: (tuple(t.shape[1:]), t.dtype) for k, t in tensors.items()}
    layout, record_bytes = _fields_layout(fields)
    rec = np.empty((n, record_bytes), dtype=np.uint8)
    for name, shape, dtype, off, nbytes in layout:
        rec[:, off:off + nbytes] = tensors[name].reshape(n, -1).view(torch.uint8).reshape(n, nbytes).numpy()
    with open(path, "wb") as f:
        f.write(rec.tobytes())
    with open(path + ".json", "w") as f:
        json.dump({"records": n, "record_bytes": record_bytes,
                   "fields": [[name, list(shape), str(dtype).replace("torch.", "")] for name, shape, dtype, _, _ in layout]}, f)
    return fields


def read_fields(path):
    """The ``fields`` mapping recorded by ``write_records`` next to ``path``."""
    with open(path + ".json") as f:
        meta = json.load(f)
    return {name: (tuple(shape), getattr(torch, dtype)) for name, shape, dtype in meta["fields"]}


class RecordFeeder:
    """Iterates over a record file in batches assembled by native background threads.

    ``fields``: name -> (shape, dtype) in record order (default: the side file of ``write_records``). Each batch is a dict
    name -> tensor ``[rows, *shape]`` viewing one of ``depth`` pinned buffers (plain host memory without CUDA); a batch stays
    valid until ``depth - 1`` further batches have been drawn, which is what a loop needs that feeds batch ``i`` and
    prefetches batch ``i + 1``. With ``world`` replicas every rank draws a disjoint, equally long part of each epoch's
    permutation. ``epochs = -1`` repeats forever.
    """

    def __init__(self, path, batch_size, fields=None, shuffle=True, seed=0, drop_last=True, depth=3, workers=2, rank=0, world=1, epochs=1,
                 pin_memory=None):
        from autodist_b200.ops import build
        self._host = build.load_host()
        self.fields = fields if fields is not None else read_fields(path)
        self._layout, self.record_bytes = _fields_layout(self.fields)
        self.batch_size = int(batch_size)
        if depth < 2:
            raise ValueError("depth must be at least 2: one batch in use, one being filled")
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        self._buffers = [torch.empty(self.batch_size * self.record_bytes, dtype=torch.uint8, pin_memory=pin) for _ in range(depth)]
        self._held = []                      # slots handed to the caller, oldest first
        self._depth = depth
        self._feeder = self._host.BatchFeeder(os.fspath(path), self.record_bytes, [(off, nb) for _, _, _, off, nb in self._layout], self.batch_size,
                                              [b.data_ptr() for b in self._buffers], workers, shuffle, seed, drop_last, rank, world, epochs)
        self.batches_per_epoch = self._feeder.batches_per_epoch
        self.records = self._feeder.records

    def __iter__(self):
        return self

    def __next__(self):
        # keep the newest depth - 1 batches alive; the oldest goes back to the workers before the next one is awaited
        while len(self._held) >= self._depth - 1:
            self._feeder.release(self._held.pop(0))
        slot = self._feeder.next()
        if slot < 0:
            raise StopIteration
        self._held.append(slot)
        rows = self._feeder.rows(slot)
        buf, out, base = self._buffers[slot], {}, 0
        for name, shape, dtype, _, nbytes in self._layout:
            block = buf[base:base + self.batch_size * nbytes][:rows * nbytes]
            out[name] = block.view(dtype).view((rows,) + shape)
            base += self.batch_size * nbytes
        return out

    def close(self):
        self._feeder.close()

    def __del__(self):
        try:
            self._feeder.close()
        except Exception:       # interpreter shutdown
            pass
