"""Session: ``sess.run(fetches, feed_dict)`` on the distributed plan.

Capability parity with ``autodist/runner.py:33-132`` (``WrappedSession``): runs
under the remapper, initialises variables on construction (replica-0 values on
every replica) and writes a Chrome trace when tracing is requested through
``RunOptions``. One session drives one rank; the other ranks execute the same
script and meet this one in the collectives.
"""
import faulthandler
import json
import os
import sys
import threading
import time

import numpy as np
import torch

from autodist_b200 import const
from autodist_b200.utils import logging, nvtx


class RunOptions:
    NO_TRACE = 0
    SOFTWARE_TRACE = 1
    HARDWARE_TRACE = 2
    FULL_TRACE = 3

    def __init__(self, trace_level=0):
        self.trace_level = trace_level


class RunMetadata:
    def __init__(self):
        self.step_stats = None
        self.trace_path = None


class _StepMetrics:
    """JSONL step metrics: step index, host and device milliseconds, samples per second, bytes all-reduced through
    the library backend, and the first scalar fetch (the loss). Device time comes from CUDA events that are read one
    step late, so enabling metrics adds no synchronisation to the step being measured."""

    def __init__(self, path, engine):
        self._path = path
        self._engine = engine
        self._cuda = engine.device.type == "cuda"
        self._step = 0
        self._pending = None
        self._bytes0 = 0
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    @classmethod
    def from_env(cls, engine):
        path = const.ENV.AUTODIST_METRICS_FILE.val
        if not path:
            return None
        if "%r" in path:
            path = path.replace("%r", str(engine.rank))
        elif engine.rank != 0:
            return None
        return cls(path, engine)

    def begin(self):
        self._flush()
        self._t0 = time.perf_counter()
        self._bytes0 = getattr(self._engine.backend, "bytes_reduced", 0)
        if self._cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()

    def end(self, result, feed_dict):
        rec = {"step": self._step, "host_ms": (time.perf_counter() - self._t0) * 1e3,
               "bytes_reduced": getattr(self._engine.backend, "bytes_reduced", 0) - self._bytes0}
        self._step += 1
        for v in (result if isinstance(result, (list, tuple)) else [result]):
            if isinstance(v, (float, np.floating)) or (isinstance(v, (np.ndarray, torch.Tensor)) and getattr(v, "size", None) is not None
                                                       and int(np.prod(tuple(v.shape))) == 1):
                rec["loss"] = float(v)
                break
        batch = next((int(v.shape[0]) for v in (feed_dict or {}).values() if hasattr(v, "shape") and len(v.shape) > 0), None)
        rec["batch"] = batch
        if self._cuda:
            self._e1.record()
            self._pending = (rec, self._e0, self._e1)
        else:
            self._write(rec, rec["host_ms"])

    def _flush(self):
        if self._pending is not None:
            rec, e0, e1 = self._pending
            self._pending = None
            e1.synchronize()
            rec["device_ms"] = e0.elapsed_time(e1)
            self._write(rec, rec["device_ms"])

    def _write(self, rec, ms):
        if rec.get("batch") and ms > 0:
            rec["samples_per_sec"] = rec["batch"] / (ms / 1e3)
        with open(self._path, "a") as f:
            f.write(json.dumps(rec) + "\n")

    def close(self):
        self._flush()


class _StepWatchdog:
    """Host-side step deadline. A daemon thread watches the running training call; when the call outlives
    ``AUTODIST_STEP_TIMEOUT`` seconds it logs the step, dumps the stack of every thread to stderr and, with
    ``AUTODIST_STEP_TIMEOUT_ACTION=abort``, ends the process with exit code 70 so that the launcher's watcher tears the
    job down (a rank stuck in a collective cannot be interrupted from Python in any other way)."""

    EXIT_CODE = 70

    def __init__(self, seconds, action="report", rank=0):
        self.seconds = float(seconds)
        self.action = action
        self.rank = rank
        self.fired = 0
        self._cond = threading.Condition()
        self._deadline = None
        self._step = None
        self._stop = False
        self._thread = threading.Thread(target=self._loop, name="autodist-step-watchdog", daemon=True)
        self._thread.start()

    @classmethod
    def from_env(cls, engine):
        raw = const.ENV.AUTODIST_STEP_TIMEOUT.val
        if not raw:
            return None
        return cls(float(raw), const.ENV.AUTODIST_STEP_TIMEOUT_ACTION.val or "report", engine.rank)

    def arm(self, step):
        with self._cond:
            self._deadline = time.monotonic() + self.seconds
            self._step = step
            self._cond.notify()

    def disarm(self):
        with self._cond:
            self._deadline = None
            self._cond.notify()

    def close(self):
        with self._cond:
            self._stop = True
            self._cond.notify()

    def _loop(self):
        with self._cond:
            while not self._stop:
                if self._deadline is None:
                    self._cond.wait()
                    continue
                left = self._deadline - time.monotonic()
                if left > 0:
                    self._cond.wait(left)
                    continue
                self.fired += 1
                self._deadline = None
                logging.error("rank %d: step %s exceeded the %.1f s deadline", self.rank, self._step, self.seconds)
                try:
                    faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
                except Exception:  # stderr may be closed during shutdown
                    pass
                if self.action == "abort":
                    os._exit(self.EXIT_CODE)


class WrappedSession:
    def __init__(self, cluster, graph_item, remapper, engine, coordinator=None, is_built=None):
        self._cluster = cluster
        self._graph_item = graph_item
        self._remapper = remapper
        self._engine = engine
        self._coordinator = coordinator
        self._is_built = is_built or (lambda: True)
        self._closed = False
        self._trace_step = 0
        self.last_step_ms = None
        self._metrics = _StepMetrics.from_env(engine)
        self._watchdog = _StepWatchdog.from_env(engine)
        logging.debug("session ready on rank %d (%s)", engine.rank, engine.device)

    @property
    def engine(self):
        return self._engine

    @property
    def remapper(self):
        return self._remapper

    @property
    def rank(self):
        return self._engine.rank

    def run(self, fetches, feed_dict=None, options=None, run_metadata=None, prefetch=None):
        """Runs one step (reference: ``autodist/runner.py`` ``WrappedSession.run``). ``prefetch``, an extension: the feed
        of the next step; its host-to-device copies start as soon as this step is launched and overlap it, and the next
        ``run`` that is fed the same value objects does not copy them again."""
        if self._closed:
            raise RuntimeError("session is closed")
        if not self._is_built():
            raise RuntimeError("the graph was modified after the distributed session was built")
        if self._coordinator is not None:
            self._coordinator.check()
        tracing = options is not None and options.trace_level > RunOptions.NO_TRACE
        if tracing:
            prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU] + (
                [torch.profiler.ProfilerActivity.CUDA] if self._engine.device.type == "cuda" else []))
            prof.__enter__()
        try:
            if self._metrics is not None:
                self._metrics.begin()
            if self._watchdog is not None:
                self._watchdog.arm(self._engine.global_step)
            try:
                with nvtx.annotate(f"step {self._engine.global_step}"):
                    result = self._run(fetches, feed_dict, prefetch)
            finally:
                if self._watchdog is not None:
                    self._watchdog.disarm()
            if self._metrics is not None:
                self._metrics.end(result, feed_dict)
        finally:
            if tracing:
                prof.__exit__(None, None, None)
                os.makedirs(const.DEFAULT_TRACE_DIR, exist_ok=True)
                path = os.path.join(const.DEFAULT_TRACE_DIR, f"timeline_{self._trace_step}.json")
                prof.export_chrome_trace(path)
                self._trace_step += 1
                if run_metadata is not None:
                    run_metadata.trace_path = path
                    run_metadata.step_stats = prof.key_averages()
        return result

    def _run(self, fetches, feed_dict, prefetch=None):
        rm, eng = self._remapper, self._engine
        single = not isinstance(fetches, (list, tuple, dict))
        leaves, rebuild = rm.flatten_fetches([fetches] if single else fetches)
        kinds = [rm.classify(l) for l in leaves]
        feeds = rm.remap_feed(feed_dict)
        tensor_idx = [i for i, k in enumerate(kinds) if k == "tensor"]
        nodes = [rm.node_of(leaves[i]) for i in tensor_idx]
        train_ops = [leaves[i] for i, k in enumerate(kinds) if k == "train_op"]
        if len(train_ops) > 1:
            from autodist_b200.parallel.engine import StepEngine
            if type(eng) is not StepEngine:
                raise NotImplementedError("several train ops in one run() call run on the generic engine only "
                                          f"(this session uses {type(eng).__name__}; on GPUs set AUTODIST_COMM=nccl)")
            values = eng.train_step_multi(train_ops, nodes, feeds)
        elif train_ops:
            values = eng.train_step(train_ops[0], nodes, feeds)
        elif nodes:
            eng.before_read()
            values = eng.forward(nodes, feeds, grad=False)
        else:
            values = []
        if prefetch is not None:
            rm.prefetch(prefetch)            # the step is launched; the next feed's copies run beside it
        out = [None] * len(leaves)
        for i, v in zip(tensor_idx, values):
            out[i] = rm.remap_fetch(v)
        for i, k in enumerate(kinds):
            if k == "variable":
                leaf = leaves[i]
                name = self._graph_item.name_of_parameter(leaf) if not isinstance(leaf, str) else (
                    leaf if leaf.endswith(":0") else leaf + ":0")
                value = eng.variable_value(name)
                if value.dtype == torch.bfloat16:
                    value = value.float()                       # numpy has no bfloat16
                out[i] = np.array(value.cpu().numpy(), copy=True)   # a copy: never a view of live parameter memory
        result = rebuild(out)
        return result[0] if single else result

    def close(self):
        if self._closed:
            return
        self._closed = True
        if self._metrics is not None:
            self._metrics.close()
        if self._watchdog is not None:
            self._watchdog.close()
        if self._coordinator is not None and getattr(self._coordinator, "failure", None) is not None:
            # a worker is known to be gone: no collective may be started on the way out
            self._engine._pending_pull = False
        try:
            self._engine.close()
        except Exception as e:  # shutting down: peers may already be gone
            logging.debug("engine close: %s", e)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
