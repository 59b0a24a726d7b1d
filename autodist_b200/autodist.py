"""User-facing facade: ``AutoDist(resource_spec_file, strategy_builder)``.

Public surface of the reference's ``autodist/autodist.py:40-322``: one instance
per process, ``scope()`` to capture a single-device program,
``create_distributed_session()`` returning a session whose
``run(fetches, feed_dict)`` executes distributed steps, ``function(fn)`` as the
decorator-style entry, ``build_strategy()`` and ``is_built()``.

Build pipeline (same order as ``autodist.py:139-150``): build or load the
strategy (the chief builds and serialises, workers load by id) -> set up the
cluster and start the other ranks -> compile the strategy -> transform into a
``DistributedPlan`` -> remapper + step engine.

Processes: one per replica device. Either the chief starts them by re-executing
the user's script (the reference's contract, via ``Coordinator``), or an external
launcher (``torchrun``) already did, in which case ``RANK`` / ``WORLD_SIZE`` are
taken from the environment and the strategy travels by broadcast.
"""
import atexit
import contextlib
import datetime
import os

import numpy as np
import torch
import torch.distributed as dist

from autodist_b200 import graph_item as _gi
from autodist_b200.cluster import SSHCluster
from autodist_b200.const import ENV
from autodist_b200.coordinator import Coordinator
from autodist_b200.graph_item import GraphItem
from autodist_b200.kernel.device.resolver import DeviceResolver
from autodist_b200.kernel.graph_transformer import GraphTransformer
from autodist_b200.remapper import Remapper
from autodist_b200.resource_spec import DeviceSpec, DeviceType, ResourceSpec
from autodist_b200.runner import WrappedSession
from autodist_b200.strategy import base
from autodist_b200.strategy.ps_strategy import PSLoadBalancing
from autodist_b200.utils import logging


def _externally_launched():
    return "RANK" in os.environ and "WORLD_SIZE" in os.environ and not ENV.AUTODIST_WORKER.val


def _is_worker():
    if ENV.AUTODIST_WORKER.val:
        return True
    return _externally_launched() and int(os.environ["RANK"]) != 0


IS_AUTODIST_WORKER = _is_worker()
IS_AUTODIST_CHIEF = not IS_AUTODIST_WORKER

_DEFAULT_AUTODIST = {}


def set_default_autodist(o):
    if os.getpid() in _DEFAULT_AUTODIST:
        raise NotImplementedError("Currently only one AutoDist instance is supported per process.")
    _DEFAULT_AUTODIST[os.getpid()] = o


def get_default_autodist():
    return _DEFAULT_AUTODIST.get(os.getpid())


def _reset_default_autodist():
    """Testing aid: forget this process's instance."""
    _DEFAULT_AUTODIST.pop(os.getpid(), None)


class AutoDist:
    def __init__(self, resource_spec_file=None, strategy_builder=None, resource_spec=None):
        set_default_autodist(self)
        self._resource_spec = resource_spec if resource_spec is not None else ResourceSpec(resource_spec_file)
        self._strategy_builder = strategy_builder or PSLoadBalancing()
        self._original_graph_item = None
        self._plan = None
        self._remapper = None
        self._session = None
        self._built_marker = None
        self._cluster = SSHCluster(self._resource_spec)
        self._coordinator = None
        self._strategy = None
        self._fn_cache = {}
        self._ph_feed_index = {}
        _gi.patch_optimizers() if ENV.AUTODIST_PATCH_TF.val else None

    # ------------------------------------------------------------------ capture
    @contextlib.contextmanager
    def scope(self):
        """Everything built inside is recorded as the single-device program to distribute."""
        if self._original_graph_item is None:
            self._original_graph_item = GraphItem()
        with self._original_graph_item.as_default():
            yield self

    @property
    def graph_item(self):
        return self._original_graph_item

    def placeholder(self, shape, dtype=torch.float32, name=None):
        return self._original_graph_item.placeholder(shape, dtype, name)

    def variable(self, initial_value, name=None, trainable=True, dtype=None):
        return self._original_graph_item.variable(initial_value, name, trainable, dtype)

    # ------------------------------------------------------------------ roles
    @property
    def rank(self):
        if _externally_launched():
            return int(os.environ["RANK"])
        if ENV.AUTODIST_WORKER.val:
            return int(ENV.AUTODIST_RANK.val)
        return self._cluster.chief_rank

    @property
    def is_chief(self):
        return not _is_worker()

    @property
    def resource_spec(self):
        return self._resource_spec

    @property
    def strategy(self):
        return self._strategy

    @property
    def plan(self):
        return self._plan

    # ------------------------------------------------------------------ build pipeline
    def build_strategy(self):
        """Strategy for the captured graph as the configured builder sees it."""
        self._original_graph_item.prepare()
        return self._strategy_builder.build(self._original_graph_item, self._resource_spec)

    def _device_for_rank(self, rank):
        spec = DeviceSpec.from_string(self._cluster.replica_devices[rank])
        if spec.device_type is DeviceType.GPU and torch.cuda.is_available():
            index = int(os.environ["LOCAL_RANK"]) if _externally_launched() and "LOCAL_RANK" in os.environ \
                else spec.device_index
            torch.cuda.set_device(index)
            return torch.device("cuda", index)
        if spec.device_type is DeviceType.GPU:
            logging.warning("replica %s requested but CUDA is unavailable: running this replica on CPU",
                            spec.name_string())
        return torch.device("cpu")

    def _init_process_group(self, device):
        world = self._cluster.world_size
        if world <= 1:
            return None
        if _externally_launched() and int(os.environ["WORLD_SIZE"]) != world:
            raise ValueError(f"WORLD_SIZE={os.environ['WORLD_SIZE']} but the resource spec has {world} replicas")
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", self._cluster.master_address)
            os.environ.setdefault("MASTER_PORT", str(self._cluster.master_port))
            timeout = datetime.timedelta(seconds=int(os.environ.get("AUTODIST_PG_TIMEOUT", "600")))
            kwargs = {}
            if device.type == "cuda":
                kwargs["device_id"] = device
            dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=self.rank,
                                    world_size=world, timeout=timeout, **kwargs)
        return dist.group.WORLD

    def _build_or_load_strategy(self):
        item = self._original_graph_item
        item.prepare()
        if _externally_launched():
            payload = [None]
            if self.rank == 0:
                s = self.build_strategy()
                s.serialize()
                payload = [s.proto.SerializeToString()]
            if self._cluster.world_size > 1:
                dist.broadcast_object_list(payload, src=0)
            from autodist_b200.proto import strategy_pb2
            msg = strategy_pb2.Strategy()
            msg.ParseFromString(payload[0])
            return base.Strategy(strategy=msg)
        if self.is_chief:
            s = self.build_strategy()
            s.serialize()
            return s
        strategy_id = ENV.AUTODIST_STRATEGY_ID.val
        assert strategy_id, "a worker needs AUTODIST_STRATEGY_ID"
        return base.Strategy.deserialize(strategy_id)

    def _compile_strategy(self, strategy):
        logging.debug("Raw strategy: %s", strategy)
        resolver = DeviceResolver(self._cluster)
        compiled = base.StrategyCompiler(self._original_graph_item) \
            .set_device_resolver(resolver.resolve_to_device_str).compile(strategy)
        logging.debug("Compiled strategy: %s", compiled)
        return compiled

    def _setup(self, strategy):
        """Chief only (and only when nobody launched the ranks for us): start the other ranks."""
        if self.is_chief and not _externally_launched() and self._cluster.world_size > 1:
            self._coordinator = Coordinator(strategy=strategy, cluster=self._cluster)
            self._cluster.start()
            self._coordinator.launch_clients()
        logging.debug("Current PID %d belongs to address %s", os.getpid(), self._cluster.get_local_address())

    def _make_engine(self, plan, device, group):
        from autodist_b200.parallel import comm
        if plan.replica.world_size <= 1:
            backend = comm.LocalBackend()
        else:
            backend = comm.TorchDistBackend(group)
        if device.type == "cuda":
            from autodist_b200.parallel.fused_engine import make_engine
            return make_engine(self._original_graph_item, plan, backend, device)
        from autodist_b200.parallel.engine import StepEngine
        return StepEngine(self._original_graph_item, plan, backend, device)

    def _build(self):
        rank = self.rank
        device = self._device_for_rank(rank)
        if _externally_launched():
            group = self._init_process_group(device)
            strategy = self._build_or_load_strategy()
        else:
            strategy = self._build_or_load_strategy()
            self._setup(strategy)
            group = self._init_process_group(device)
        self._strategy = strategy
        compiled = self._compile_strategy(strategy)
        transformer = GraphTransformer(compiled, self._cluster, self._original_graph_item, rank=rank)
        self._plan = transformer.transform()
        local_group = None
        if self._plan.replica.num_workers > 1:
            for host in self._cluster.nodes:
                ranks = self._cluster.ranks_of_node(host)
                g = dist.new_group(ranks)
                if rank in ranks:
                    local_group = g
        engine = self._make_engine(self._plan, device, group)
        self._remapper = Remapper(self._original_graph_item, self._plan, device, local_group)
        self._built_marker = len(self._original_graph_item.tracer.graph.nodes)
        return engine

    def is_built(self):
        if self._session is None:
            return False
        if ENV.AUTODIST_IS_TESTING.val:
            # the captured graph must not grow after the plan was made from it
            return len(self._original_graph_item.tracer.graph.nodes) == self._built_marker
        return True

    def _create_distributed_session(self):
        if self._session is None:
            engine = self._build()
            self._session = WrappedSession(self._cluster, self._original_graph_item, self._remapper, engine,
                                           coordinator=self._coordinator, is_built=self._is_current)
            atexit.register(self._shutdown)
        return self._session

    def _is_current(self):
        if ENV.AUTODIST_IS_TESTING.val and self._built_marker is not None:
            return len(self._original_graph_item.tracer.graph.nodes) == self._built_marker
        return True

    def create_distributed_session(self):
        """Build (on first call) and return the session that executes the captured graph."""
        return self._create_distributed_session()

    def _shutdown(self):
        if self._session is not None:
            self._session.close()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception as e:  # peers may already be gone
                logging.debug("destroy_process_group: %s", e)
        if self._coordinator is not None:
            try:
                self._coordinator.join(timeout=30)
            except Exception as e:
                logging.error("%s", e)

    # ------------------------------------------------------------------ function-style entry
    def _args_to_placeholders(self, args, kwargs):
        item = self._original_graph_item

        def convert(v, index):
            if isinstance(v, (np.ndarray, torch.Tensor)) and v.ndim >= 1:
                logging.debug("treating dimension 0 of function input %s as the batch dimension", tuple(v.shape))
                dtype = v.dtype if isinstance(v, torch.Tensor) else torch.from_numpy(np.zeros(0, v.dtype)).dtype
                if dtype == torch.float64:
                    dtype = torch.float32
                ph = item.placeholder((None,) + tuple(v.shape[1:]), dtype)
                self._ph_feed_index[ph] = index
                return ph
            return v

        return tuple(convert(a, i) for i, a in enumerate(args)), {k: convert(v, k) for k, v in kwargs.items()}

    def function(self, fn):
        """Decorator: the first call traces ``fn`` (array arguments become batch-split placeholders),
        builds the session and afterwards every call is one ``session.run``."""
        def wrapper(*args, **kwargs):
            if fn not in self._fn_cache:
                if self._fn_cache:
                    raise NotImplementedError("AutoDist currently only stably supports one "
                                              "'autodist.function' across the scope.")
                ph_args, ph_kwargs = None, None
                ctx = contextlib.nullcontext() if _gi.get_default_graph_item() is self._original_graph_item \
                    else self.scope()
                with ctx:
                    ph_args, ph_kwargs = self._args_to_placeholders(args, kwargs)
                    fetches = fn(*ph_args, **ph_kwargs)
                session = self._create_distributed_session()
                index = dict(self._ph_feed_index)

                def run_fn(*a, **kw):
                    feed = {ph: (a[i] if isinstance(i, int) else kw[i]) for ph, i in index.items()}
                    return session.run(fetches, feed)

                self._fn_cache[fn] = run_fn
            return self._fn_cache[fn](*args, **kwargs)
        return wrapper
