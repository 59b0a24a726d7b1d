"""Small training-loop utilities shared by the example drivers.

They stand in for the vendored helper tree of the reference's examples:

* ``TimeHistory`` - examples/s per logging window (reference: ``examples/benchmark/utils/misc/keras_utils.py:41-99``);
* ``MetricsLogger`` - one JSON object per line (reference: ``examples/benchmark/utils/logs/logger.py:108-300`` without the
  BigQuery / MLPerf back ends);
* ``warmup_linear_decay`` / ``PiecewiseConstantDecayWithWarmup`` - learning-rate schedules
  (reference: ``examples/benchmark/utils/common.py:28-67,112-179``);
* ``add_*_flags`` - the argparse equivalent of the absl flag groups (reference: ``examples/benchmark/utils/flags/_base.py``,
  ``_performance.py``, ``_benchmark.py``).

The schedules return plain multipliers / values so they can be written into the device-resident learning-rate tensor
of a fused optimizer between steps without re-capturing a CUDA graph.
"""
import json
import os
import time
from bisect import bisect_right


class TimeHistory:
    """Per-window throughput bookkeeping for a hand-written training loop.

    ``on_step_end()`` returns a record every ``log_steps`` steps: ``{"step", "elapsed_s", "examples_per_sec"}``.
    The caller decides whether to synchronise the device first; an asynchronous loop measures launch rate otherwise.
    """

    def __init__(self, batch_size, log_steps=100, clock=time.perf_counter):
        self.batch_size = int(batch_size)
        self.log_steps = max(1, int(log_steps))
        self._clock = clock
        self.global_step = 0
        self.records = []
        self._window_start = None
        self._train_start = None

    def on_train_begin(self):
        self._train_start = self._window_start = self._clock()

    def on_step_end(self):
        if self._window_start is None:
            self.on_train_begin()
        self.global_step += 1
        if self.global_step % self.log_steps:
            return None
        now = self._clock()
        elapsed = now - self._window_start
        rec = {"step": self.global_step, "elapsed_s": elapsed,
               "examples_per_sec": self.batch_size * self.log_steps / elapsed if elapsed > 0 else float("inf")}
        self.records.append(rec)
        self._window_start = now
        return rec

    @property
    def average_examples_per_sec(self):
        """Mean over the windows after the first (which contains warm-up and graph capture)."""
        recs = self.records[1:] or self.records
        if not recs:
            return 0.0
        return sum(r["examples_per_sec"] for r in recs) / len(recs)


class MetricsLogger:
    """Append-only JSONL metric sink: ``log_metric(name, value, unit, global_step, extras)``; ``log_run_info`` once."""

    def __init__(self, path=None, stream=None):
        self._path = path
        self._stream = stream
        if path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def _emit(self, obj):
        line = json.dumps(obj, sort_keys=True)
        if self._path:
            with open(self._path, "a") as f:
                f.write(line + "\n")
        if self._stream is not None:
            print(line, file=self._stream, flush=True)

    def log_run_info(self, model_name, dataset_name, run_params=None):
        self._emit({"kind": "run_info", "model_name": model_name, "dataset": dataset_name,
                    "run_parameters": dict(run_params or {}), "timestamp": time.time()})

    def log_metric(self, name, value, unit=None, global_step=None, extras=None):
        try:
            value = float(value)
        except (TypeError, ValueError):
            return False                                                      # non-numeric metrics are dropped, not fatal
        self._emit({"kind": "metric", "name": name, "value": value, "unit": unit, "global_step": global_step,
                    "extras": dict(extras or {}), "timestamp": time.time()})
        return True


def warmup_linear_decay(step, base_lr, total_steps, warmup_steps=0, end_lr=0.0):
    """BERT schedule: linear warm-up to ``base_lr`` over ``warmup_steps`` then linear decay to ``end_lr``."""
    if warmup_steps and step < warmup_steps:
        return base_lr * (step + 1) / warmup_steps
    frac = min(1.0, max(0.0, (step - warmup_steps) / max(1, total_steps - warmup_steps)))
    return base_lr + (end_lr - base_lr) * frac


class PiecewiseConstantDecayWithWarmup:
    """ImageNet schedule: linear warm-up over ``warmup_epochs`` then a step function over epoch boundaries.

    ``base_lr`` is scaled by ``batch_size / base_batch`` (the usual 0.1 per 256 images rule).
    """

    def __init__(self, batch_size, epoch_size, warmup_epochs, boundaries, multipliers, base_lr=0.1, base_batch=256):
        if len(boundaries) != len(multipliers) - 1:
            raise ValueError("need exactly one more multiplier than boundaries")
        self.rescaled_lr = base_lr * batch_size / base_batch
        self.steps_per_epoch = max(1, epoch_size // batch_size)
        self.warmup_steps = warmup_epochs * self.steps_per_epoch
        self.step_boundaries = [self.steps_per_epoch * b for b in boundaries]
        self.lr_values = [self.rescaled_lr * m for m in multipliers]

    def __call__(self, step):
        if step < self.warmup_steps:
            return self.rescaled_lr * step / self.warmup_steps
        return self.lr_values[bisect_right(self.step_boundaries, step)]


def set_learning_rate(optimizer, lr):
    """Write ``lr`` into every parameter group; tensor-valued learning rates (graph-safe) are filled in place."""
    for group in optimizer.param_groups:
        cur = group.get("lr")
        if hasattr(cur, "fill_"):
            cur.fill_(lr)
        else:
            group["lr"] = lr


def add_base_flags(parser, batch_size=32, train_steps=100):
    g = parser.add_argument_group("base")
    g.add_argument("--batch_size", type=int, default=batch_size, help="per-GPU batch size")
    g.add_argument("--train_steps", type=int, default=train_steps)
    g.add_argument("--model_dir", default=None, help="checkpoint / metrics directory")
    g.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    g.add_argument("--resource_spec", default=None, help="resource-spec YAML; default is this node's GPUs")
    return g


def add_performance_flags(parser):
    g = parser.add_argument_group("performance")
    g.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    g.add_argument("--use_synthetic_data", action="store_true", default=True)
    g.add_argument("--cuda_graph", type=int, default=1, help="capture the whole step in a CUDA graph")
    g.add_argument("--flight_mb", type=int, default=None, help="gradient flight size for the fused all-reduce")
    return g


def add_benchmark_flags(parser, log_steps=100):
    g = parser.add_argument_group("benchmark")
    g.add_argument("--log_steps", type=int, default=log_steps)
    g.add_argument("--benchmark_log", default=None, help="JSONL metrics file")
    return g


def add_strategy_flags(parser, default="AllReduce"):
    g = parser.add_argument_group("distribution")
    g.add_argument("--autodist_strategy", default=default,
                   choices=["PS", "PSLoadBalancing", "PartitionedPS", "UnevenPartitionedPS", "AllReduce", "PartitionedAR",
                            "RandomAxisPartitionAR", "Parallax", "Auto"])
    g.add_argument("--chunk_size", type=int, default=256)
    g.add_argument("--compressor", default="NoneCompressor",
                   choices=["NoneCompressor", "HorovodCompressor", "HorovodCompressorEF", "PowerSGDCompressor"])
    return g


def build_strategy(name, chunk_size=256, compressor="NoneCompressor", num_gpus=1):
    """Strategy builder from the ``--autodist_strategy`` family of flags."""
    from autodist_b200 import strategy as S
    ar = dict(chunk_size=chunk_size, compressor=compressor)
    table = {
        "PS": lambda: S.PS(), "PSLoadBalancing": lambda: S.PSLoadBalancing(),
        "PartitionedPS": lambda: S.PartitionedPS(), "UnevenPartitionedPS": lambda: S.UnevenPartitionedPS(),
        "AllReduce": lambda: S.AllReduce(**ar), "PartitionedAR": lambda: S.PartitionedAR(chunk_size=chunk_size),
        "RandomAxisPartitionAR": lambda: S.RandomAxisPartitionAR(chunk_size=chunk_size),
        "Parallax": lambda: S.Parallax(**ar), "Auto": lambda: S.AutoStrategy(),
    }
    if name not in table:
        raise ValueError(f"unknown strategy {name!r}")
    return table[name]()
