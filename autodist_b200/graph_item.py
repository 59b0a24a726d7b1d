"""Graph capture: the single-device program the user writes inside ``ad.scope()``.

Capability parity with the reference's ``autodist/graph_item.py:73-553`` (a
wrapper of the user's graph plus variable / gradient / optimizer / saver
records, with a proto round-trip), rebuilt over ``torch.fx``:

* placeholders are fx ``placeholder`` nodes handed to the user as symbolic
  tensors; running ordinary ``nn.Module`` / ``torch`` code on them records
  ``call_function`` / ``call_method`` nodes, parameters become ``get_attr``
  nodes of a container module owned by the item;
* modules flagged ``_autodist_leaf = True`` are recorded as one ``call_module``
  node (their forward then runs eagerly with hand-written CUDA ops inside);
* ``torch.optim.Optimizer.__init__`` is wrapped so that the optimizer class,
  its constructor arguments and its parameter groups are captured (reference:
  ``graph_item.py:73-109`` wrapping ``__init__`` / ``apply_gradients``), and
  ``optimizer.minimize(loss)`` returns the ``train_op`` handle and records the
  gradient -> variable pairs.
"""
import contextlib
import functools
import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.fx as fx
from torch import nn

from autodist_b200.proto import graphitem_pb2
from autodist_b200.utils import logging

_default_graph_item = None
_capture_suspended = 0


@contextlib.contextmanager
def suspend_capture():
    """Objects created inside (e.g. the engine's per-shard optimizers) are not recorded."""
    global _capture_suspended
    _capture_suspended += 1
    try:
        yield
    finally:
        _capture_suspended -= 1


def get_default_graph_item():
    return _default_graph_item


def _dtype_size(dtype):
    return torch.empty((), dtype=dtype).element_size()


@dataclass
class VariableInfo:
    """What a strategy builder may know about one variable."""
    name: str                    # "<qualified.name>:0"
    shape: Tuple[int, ...]
    dtype: torch.dtype
    trainable: bool = True
    sparse_grad: bool = False    # gradient is (indices, values) rows, never densified
    in_control_flow: bool = False
    path: str = ""               # attribute path below the item's container module

    @property
    def op_name(self):
        return self.name[:-2] if self.name.endswith(":0") else self.name

    @property
    def numel(self):
        n = 1
        for d in self.shape:
            n *= int(d)
        return n

    @property
    def byte_size(self):
        return self.numel * _dtype_size(self.dtype)

    def to_record(self):
        return {"name": self.name, "shape": list(self.shape), "dtype": str(self.dtype),
                "trainable": self.trainable, "sparse_grad": self.sparse_grad,
                "in_control_flow": self.in_control_flow}

    @classmethod
    def from_record(cls, rec):
        return cls(rec["name"], tuple(rec["shape"]), getattr(torch, rec["dtype"].split(".")[-1]),
                   rec["trainable"], rec["sparse_grad"], rec["in_control_flow"])


@dataclass
class PlaceholderInfo:
    name: str
    shape: Tuple[Optional[int], ...]
    dtype: torch.dtype

    @property
    def batch_dim(self):
        """Index of the polymorphic (``None``) dimension that feeds are split on, or ``None``."""
        for i, d in enumerate(self.shape):
            if d is None:
                return i
        return None


@dataclass
class OptimizerInfo:
    optimizer: Any
    cls: type
    args: tuple
    kwargs: dict
    name: str


class TrainOp:
    """Handle returned by ``optimizer.minimize(loss)``; fetch it to take one training step."""

    def __init__(self, item, optimizer_index, loss_node, var_list=None, clip_global_norm=None, name="train_op"):
        self.item = item
        self.optimizer_index = optimizer_index
        self.loss_node = loss_node
        self.var_list = var_list
        self.clip_global_norm = clip_global_norm  # (max_norm, [parameters]) or None
        self.name = name

    def __repr__(self):
        return f"<TrainOp {self.name} loss={self.loss_node.name}>"


_CONTROL_FLOW_HINT = ("a captured tensor decides a Python branch or loop here (data-dependent control flow). Code inside an nn.Module "
                      "is handled automatically: the module is recorded as one opaque node and its variables are marked "
                      "in_control_flow (never partitioned). Code written directly in the scope has to move into a module.")


class SymbolicTensor(fx.Proxy):
    """An fx proxy usable as a ``feed_dict`` key / fetch handle."""

    def __hash__(self):
        return id(self)

    def _needs_value(self, *_):
        raise fx.proxy.TraceError(_CONTROL_FLOW_HINT)

    # every way Python can ask a tensor for a concrete value while the program is only being recorded
    __bool__ = __float__ = __int__ = __index__ = __len__ = __iter__ = item = tolist = _needs_value

    @property
    def op_name(self):
        return self.node.name


class _CaptureTracer(fx.Tracer):
    def __init__(self, item):
        super().__init__()
        self.item = item
        self.root = item.root
        self.graph = fx.Graph(tracer_cls=type(self))
        self.tensor_attrs = {}
        self.submodule_paths = None
        self.module_stack = {}
        self.node_name_to_scope = {}
        self.scope = fx.proxy.Scope("", None)
        self._attr_nodes: Dict[str, fx.Node] = {}

    def proxy(self, node):
        return SymbolicTensor(node, self)

    def _get_attr_node(self, path):
        node = self._attr_nodes.get(path)
        if node is None:
            node = self.create_node("get_attr", path, (), {})
            self._attr_nodes[path] = node
        return node

    def create_arg(self, a):
        if isinstance(a, nn.Parameter):
            return self._get_attr_node(self.item.path_of_parameter(a))
        if isinstance(a, torch.Tensor) and not isinstance(a, fx.Proxy):
            path = self.item.path_of_buffer(a)
            return self._get_attr_node(path)
        return super().create_arg(a)


def _contains_proxy(obj):
    if isinstance(obj, fx.Proxy):
        return True
    if isinstance(obj, (list, tuple)):
        return any(_contains_proxy(o) for o in obj)
    if isinstance(obj, dict):
        return any(_contains_proxy(o) for o in obj.values())
    return False


def graph_op(fn):
    """Make ``fn`` (e.g. an ``autograd.Function`` wrapper around a CUDA kernel) recordable.

    Called with symbolic tensors it adds one ``call_function`` node to the graph
    being captured; called with real tensors it just runs.
    """
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if _contains_proxy(args) or _contains_proxy(kwargs):
            item = get_default_graph_item()
            if item is None:
                raise RuntimeError(f"{fn.__name__} received a symbolic tensor outside ad.scope()")
            return item.tracer.create_proxy("call_function", wrapper, args, kwargs)
        return fn(*args, **kwargs)
    wrapper.__graph_op__ = True
    return wrapper


class GraphItem:
    """The captured program plus the records the strategy builders and transformer passes query."""

    def __init__(self, name="graph"):
        self.name = name
        self.root = nn.Module()          # container: tracked modules + bare parameters + constants
        self.tracer = _CaptureTracer(self)
        self.placeholders: Dict[str, PlaceholderInfo] = {}
        self._placeholder_proxies: Dict[str, SymbolicTensor] = {}
        self.optimizers: List[OptimizerInfo] = []
        self.train_ops: List[TrainOp] = []
        self.grad_target_pairs: Dict[str, str] = {}
        self.savers: List[Any] = []
        self.table_initializers: List[str] = []
        self._tracked_modules: List[nn.Module] = []
        self._module_prefix: Dict[int, str] = {}
        self._param_paths: Dict[int, str] = {}
        self._param_names: Dict[int, str] = {}
        self._buffer_paths: Dict[int, str] = {}
        self._named_bare: Dict[str, nn.Parameter] = {}
        self._sparse_params = set()
        self._control_flow_params = set()      # ids of parameters of modules whose forward branches on tensor values
        self._variables: Optional[Dict[str, VariableInfo]] = None
        self._prepared = False
        self._frozen_record = None       # set on a deserialized (description-only) item

    # ------------------------------------------------------------------ context
    @contextlib.contextmanager
    def as_default(self):
        global _default_graph_item
        if _default_graph_item is not None:
            raise SyntaxError("GraphItem does not support nested contexts.")
        _default_graph_item = self
        unpatch = _patch_module_capture(self)
        try:
            yield self
        finally:
            unpatch()
            _default_graph_item = None

    # ------------------------------------------------------------------ capture API
    def placeholder(self, shape, dtype=torch.float32, name=None):
        if name is None:
            name = "Placeholder" if not self.placeholders else f"Placeholder_{len(self.placeholders)}"
        if name in self.placeholders:
            raise ValueError(f"duplicate placeholder name {name!r}")
        self.placeholders[name] = PlaceholderInfo(name, tuple(shape), dtype)
        proxy = self.tracer.create_proxy("placeholder", name, (), {})
        self._placeholder_proxies[name] = proxy
        self._variables = None
        return proxy

    def variable(self, initial_value, name=None, trainable=True, dtype=None):
        """A bare named variable (TF-style). Returns an ``nn.Parameter`` registered on the item."""
        t = torch.as_tensor(initial_value, dtype=dtype).clone().detach()
        if not t.is_floating_point():
            trainable = False
        p = nn.Parameter(t, requires_grad=trainable)
        base = name or "Variable"
        cand, k = base, 0
        while cand in self._named_bare:
            k += 1
            cand = f"{base}_{k}"
        self._named_bare[cand] = p
        self._register_parameter(p, cand, "v__" + cand.replace(".", "_").replace("/", "_"))
        return p

    def track_module(self, module):
        """Remember a module constructed in scope; roots are resolved in ``prepare``."""
        self._tracked_modules.append(module)

    def mark_sparse(self, param):
        """Declare that ``param`` receives row-sparse gradients (embedding-style lookups)."""
        self._sparse_params.add(id(param))
        self._variables = None

    # ------------------------------------------------------------------ parameter naming
    def _register_parameter(self, p, name, path):
        self._param_paths[id(p)] = path
        self._param_names[id(p)] = name + ":0"
        if "." not in path:
            self.root.register_parameter(path, p)
        self._variables = None

    def _root_modules(self):
        tracked = [m for m in self._tracked_modules]
        children = set()
        for m in tracked:
            for sub in m.modules():
                if sub is not m:
                    children.add(id(sub))
        roots, seen = [], set()
        for m in tracked:
            if id(m) not in children and id(m) not in seen:
                seen.add(id(m))
                if any(True for _ in m.parameters()) or any(True for _ in m.buffers()):
                    roots.append(m)
        return roots

    def _refresh_module_registry(self):
        roots = self._root_modules()
        single = len(roots) == 1
        counts: Dict[str, int] = {}
        for m in roots:
            if id(m) in self._module_prefix:
                continue
            attr = f"m{len(self._module_prefix)}"
            if single:
                prefix = ""
            else:
                base = type(m).__name__.lower()
                k = counts.get(base, sum(1 for v in self._module_prefix.values() if v.startswith(base)))
                counts[base] = k + 1
                prefix = f"{base}_{k}/" if k else f"{base}/"
            self._module_prefix[id(m)] = prefix
            self.root.add_module(attr, m)
            for pname, p in m.named_parameters():
                if id(p) not in self._param_paths:
                    self._param_paths[id(p)] = f"{attr}.{pname}"
                    self._param_names[id(p)] = f"{prefix}{pname}:0"
            for bname, b in m.named_buffers():
                self._buffer_paths.setdefault(id(b), f"{attr}.{bname}")
        self._variables = None

    def path_of_parameter(self, p):
        path = self._param_paths.get(id(p))
        if path is None:
            self._refresh_module_registry()
            path = self._param_paths.get(id(p))
        if path is None:
            # A bare parameter the user created without ad.variable(): TF-style default naming.
            k = sum(1 for n in self._named_bare if n.startswith("Variable"))
            name = "Variable" if k == 0 else f"Variable_{k}"
            self._named_bare[name] = p
            self._register_parameter(p, name, "v__" + name)
            path = self._param_paths[id(p)]
        return path

    def path_of_buffer(self, t):
        path = self._buffer_paths.get(id(t))
        if path is None:
            self._refresh_module_registry()
            path = self._buffer_paths.get(id(t))
        if path is None:
            path = f"_tensor_constant{len(self._buffer_paths)}"
            self.root.register_buffer(path, t, persistent=False)
            self._buffer_paths[id(t)] = path
        return path

    def path_of_module(self, module):
        for name, m in self.root.named_modules():
            if m is module:
                return name
        self._refresh_module_registry()
        for name, m in self.root.named_modules():
            if m is module:
                return name
        # A leaf module constructed outside the tracked set: adopt it.
        self._tracked_modules.append(module)
        self._refresh_module_registry()
        for name, m in self.root.named_modules():
            if m is module:
                return name
        raise KeyError("module is not reachable from the captured graph")

    def name_of_parameter(self, p):
        self.path_of_parameter(p)
        return self._param_names[id(p)]

    # ------------------------------------------------------------------ optimizer capture
    def extend_optimizer_info(self, optimizer, args, kwargs):
        # `kwargs` are the defaults the base class received; keep those the subclass's constructor accepts (a subclass may pass
        # its parent more than it takes itself: AdamW hands Adam `decoupled_weight_decay`), so that the engines can build
        # the same optimizer again over their own parameter objects
        import inspect
        accepted = inspect.signature(type(optimizer).__init__).parameters
        if not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in accepted.values()):
            kwargs = {k: v for k, v in kwargs.items() if k in accepted}
        self.optimizers.append(OptimizerInfo(optimizer, type(optimizer), args, kwargs,
                                             f"{type(optimizer).__name__}_{len(self.optimizers)}"))
        for group in optimizer.param_groups:
            for p in group["params"]:
                self.path_of_parameter(p)
        self._variables = None

    def _optimizer_index(self, optimizer):
        for i, info in enumerate(self.optimizers):
            if info.optimizer is optimizer:
                return i
        raise ValueError("optimizer was not constructed inside ad.scope()")

    def extend_gradient_info(self, optimizer, loss, var_list=None, clip_global_norm=None):
        if not isinstance(loss, fx.Proxy):
            raise TypeError("minimize() expects the symbolic loss built from placeholders inside ad.scope()")
        idx = self._optimizer_index(optimizer)
        op = TrainOp(self, idx, loss.node, var_list, clip_global_norm, name=f"train_op_{len(self.train_ops)}")
        self.train_ops.append(op)
        params = var_list if var_list is not None else [p for g in optimizer.param_groups for p in g["params"]]
        reachable = self._params_reaching(loss.node)
        for p in params:
            if id(p) in reachable and p.requires_grad:
                vname = self.name_of_parameter(p)
                self.grad_target_pairs[f"gradients/{vname[:-2]}_grad:0"] = vname
        self._variables = None
        return op

    def _params_reaching(self, node):
        """ids of parameters that are ancestors of ``node`` in the captured graph."""
        by_path = {path: pid for pid, path in self._param_paths.items()}
        seen, stack, found = set(), [node], set()
        while stack:
            n = stack.pop()
            if n in seen:
                continue
            seen.add(n)
            if n.op == "get_attr" and n.target in by_path:
                found.add(by_path[n.target])
            elif n.op == "call_module":
                mod = self.root.get_submodule(n.target)
                for p in mod.parameters():
                    self.path_of_parameter(p)
                    found.add(id(p))
            stack.extend(n.all_input_nodes)
        return found

    def mark_control_flow(self, module):
        """``module`` runs as an opaque node because its forward depends on tensor values: its variables must stay whole."""
        for p in module.parameters():
            self._control_flow_params.add(id(p))
        self._variables = None

    # ------------------------------------------------------------------ queries used by builders / passes
    def prepare(self):
        """Freeze the naming registry and detect sparse-gradient variables."""
        self._refresh_module_registry()
        for m in list(self.root.modules()):
            if isinstance(m, nn.Embedding) and m.sparse:
                self._sparse_params.add(id(m.weight))
            for p in getattr(m, "sparse_grad_parameters", lambda: [])():
                self._sparse_params.add(id(p))
            if getattr(m, "_autodist_control_flow", False):          # a leaf module may declare it itself
                self.mark_control_flow(m)
        self._variables = None
        self._prepared = True
        return self

    def _all_parameters(self):
        out, seen = [], set()
        for info in self.optimizers:
            for g in info.optimizer.param_groups:
                for p in g["params"]:
                    if id(p) not in seen:
                        seen.add(id(p))
                        out.append(p)
        for _, p in self.root.named_parameters():
            if id(p) not in seen:
                seen.add(id(p))
                out.append(p)
        return out

    @property
    def variables(self):
        """``name -> VariableInfo`` of every parameter known to the item (trainable or not)."""
        if self._frozen_record is not None:
            return {r["name"]: VariableInfo.from_record(r) for r in self._frozen_record["variables"]}
        if self._variables is None:
            self._refresh_module_registry()
            out = {}
            for p in self._all_parameters():
                name = self.name_of_parameter(p)
                out[name] = VariableInfo(name, tuple(p.shape), p.dtype, p.requires_grad,
                                         id(p) in self._sparse_params, id(p) in self._control_flow_params, self._param_paths[id(p)])
            self._variables = out
        return self._variables

    @property
    def trainable_var_op_to_var(self):
        """``op name -> VariableInfo`` for trainable variables, in optimizer / declaration order."""
        return {v.op_name: v for v in self.variables.values() if v.trainable}

    def updated_variable_names(self):
        """Names of variables that have a gradient -> update (the rest is pruned by the compiler)."""
        return set(self.grad_target_pairs.values())

    @property
    def var_op_name_to_grad_info(self):
        """``op name -> (gradient name, variable, update-op name)`` for every updated variable."""
        out = {}
        for gname, vname in self.grad_target_pairs.items():
            var = self.variables[vname]
            opt = self._optimizer_of(vname)
            out[var.op_name] = (gname, var, f"{opt}/update_{var.op_name}")
        return out

    def _optimizer_of(self, var_name):
        for info in self.optimizers:
            for g in info.optimizer.param_groups:
                for p in g["params"]:
                    if self._param_names.get(id(p)) == var_name:
                        return info.name
        return "optimizer"

    def parameter_by_name(self, name):
        for p in self._all_parameters():
            if self._param_names.get(id(p)) == name:
                return p
        raise KeyError(name)

    def named_parameters(self):
        """(``name:0``, parameter) in variable order."""
        return [(self.name_of_parameter(p), p) for p in self._all_parameters()]

    def named_buffers(self):
        out = []
        for m_attr, m in self.root.named_children():
            prefix = self._module_prefix.get(id(m), "")
            for bname, b in m.named_buffers():
                out.append((f"{prefix}{bname}", b))
        return out

    def placeholder_of(self, key):
        """Resolve a feed key (symbolic tensor or name) to its ``PlaceholderInfo``."""
        if isinstance(key, fx.Proxy):
            key = key.node.target if key.node.op == "placeholder" else key.node.name
        if isinstance(key, str):
            key = key[:-2] if key.endswith(":0") else key
            if key in self.placeholders:
                return self.placeholders[key]
        raise KeyError(f"{key!r} is not a placeholder of this graph")

    def update_savers(self, saver):
        self.savers.append(saver)

    # ------------------------------------------------------------------ compilation of fetch sets
    def compile_fetches(self, nodes):
        """A ``GraphModule`` computing ``nodes`` (tuple) from the placeholders they depend on."""
        graph = fx.Graph()
        env = {}
        needed, stack = set(), list(nodes)
        while stack:
            n = stack.pop()
            if n in needed:
                continue
            needed.add(n)
            stack.extend(n.all_input_nodes)
        used_placeholders = []
        for n in self.tracer.graph.nodes:
            if n not in needed:
                continue
            env[n] = graph.node_copy(n, lambda x: env[x])
            if n.op == "placeholder":
                used_placeholders.append(n.target)
        graph.output(tuple(env[n] for n in nodes))
        gm = fx.GraphModule(self.root, graph)
        return gm, used_placeholders

    def graph_text(self):
        if self._frozen_record is not None:
            return self._frozen_record["graph"]
        return str(self.tracer.graph)

    # ------------------------------------------------------------------ proto round trip
    def _record(self):
        return {
            "graph": self.graph_text(),
            "placeholders": [{"name": p.name, "shape": list(p.shape), "dtype": str(p.dtype)}
                             for p in self.placeholders.values()] if self._frozen_record is None
            else self._frozen_record["placeholders"],
            "variables": [v.to_record() for v in self.variables.values()],
            "optimizers": [{"name": o.name, "cls": f"{o.cls.__module__}.{o.cls.__qualname__}",
                            "kwargs": {k: repr(v) for k, v in o.kwargs.items()}} for o in self.optimizers]
            if self._frozen_record is None else self._frozen_record["optimizers"],
        }

    def serialize(self, path=None):
        from google.protobuf import wrappers_pb2
        rec = self._record()
        msg = graphitem_pb2.GraphItem()
        msg.graph_def.Pack(wrappers_pb2.BytesValue(value=json.dumps(
            {k: rec[k] for k in ("graph", "placeholders", "optimizers")}).encode()))
        for gname, vname in self.grad_target_pairs.items():
            msg.grad_target_pairs[gname] = vname
        for v in rec["variables"]:
            msg.info.variables.add().Pack(wrappers_pb2.BytesValue(value=json.dumps(v).encode()))
        msg.info.table_initializers.extend(self.table_initializers)
        for s in self.savers:
            msg.info.savers.add().Pack(wrappers_pb2.BytesValue(value=json.dumps(
                getattr(s, "saver_def", lambda: {})()).encode()))
        data = msg.SerializeToString()
        if path is not None:
            with open(path, "wb") as f:
                f.write(data)
        return data

    @classmethod
    def deserialize(cls, data_or_path):
        from google.protobuf import wrappers_pb2
        if isinstance(data_or_path, (bytes, bytearray)):
            data = bytes(data_or_path)
        else:
            with open(data_or_path, "rb") as f:
                data = f.read()
        msg = graphitem_pb2.GraphItem()
        msg.ParseFromString(data)
        item = cls()
        holder = wrappers_pb2.BytesValue()
        msg.graph_def.Unpack(holder)
        rec = json.loads(holder.value.decode())
        rec["variables"] = []
        for any_msg in msg.info.variables:
            any_msg.Unpack(holder)
            rec["variables"].append(json.loads(holder.value.decode()))
        item._frozen_record = rec
        item.grad_target_pairs = dict(msg.grad_target_pairs)
        item.table_initializers = list(msg.info.table_initializers)
        return item

    def __eq__(self, other):
        return (isinstance(other, GraphItem) and self._record() == other._record()
                and self.grad_target_pairs == other.grad_target_pairs)

    __hash__ = object.__hash__


# ---------------------------------------------------------------------- patches
_optimizer_patched = False


def patch_optimizers():
    """Wrap ``torch.optim.Optimizer.__init__`` (once per process) and add ``minimize``.

    Every ``torch.optim`` subclass funnels through the base ``__init__``, so one
    wrapper sees them all (the reference walks the subclass tree instead,
    ``patch.py:79-88``). Capture only happens while a graph item is the default.
    """
    global _optimizer_patched
    if _optimizer_patched:
        return
    _optimizer_patched = True
    base_init = torch.optim.Optimizer.__init__

    @functools.wraps(base_init)
    def wrapped_init(self, params, defaults):
        base_init(self, params, defaults)
        item = get_default_graph_item()
        if item is not None and not _capture_suspended:
            item.extend_optimizer_info(self, (), dict(defaults))

    torch.optim.Optimizer.__init__ = wrapped_init

    def minimize(self, loss, var_list=None, clip_global_norm=None):
        """``train_op`` for ``loss``; ``clip_global_norm=(max_norm, [parameters])`` clips those gradients jointly."""
        item = get_default_graph_item()
        if item is None:
            raise RuntimeError("optimizer.minimize(loss) must be called inside ad.scope()")
        return item.extend_gradient_info(self, loss, var_list, clip_global_norm)

    torch.optim.Optimizer.minimize = minimize


# Library modules whose forward branches on its inputs (dimension checks, packed sequences, masks): recorded as one
# node instead of being traced through. User modules opt in with ``_autodist_leaf = True``.
_AUTO_LEAF_MODULES = (nn.RNNBase, nn.RNNCellBase, nn.MultiheadAttention, nn.TransformerEncoderLayer,
                      nn.TransformerDecoderLayer, nn.TransformerEncoder, nn.TransformerDecoder, nn.Transformer)


def _patch_module_capture(item):
    """While ``item`` is the default: track constructed modules, and record leaf modules as one node."""
    orig_init = nn.Module.__init__
    orig_call = nn.Module.__call__

    @functools.wraps(orig_init)
    def tracking_init(self, *args, **kwargs):
        orig_init(self, *args, **kwargs)
        if self is not item.root and not _capture_suspended:
            item.track_module(self)

    @functools.wraps(orig_call)
    def leaf_call(self, *args, **kwargs):
        symbolic = _contains_proxy(args) or _contains_proxy(kwargs)
        if (getattr(self, "_autodist_leaf", False) or isinstance(self, _AUTO_LEAF_MODULES)) and symbolic:
            return item.tracer.create_proxy("call_module", item.path_of_module(self), args, kwargs)
        if not symbolic or self is item.root:
            return orig_call(self, *args, **kwargs)
        # Trace through the module; if its forward turns out to branch or loop on tensor values (the reference's
        # tf.cond / tf.while_loop cases, tests/integration/cases/c2.py:50-52, c4.py:31), undo what the attempt recorded,
        # record the module as one opaque node instead, and mark its variables so that no builder partitions them.
        graph = item.tracer.graph
        mark = len(graph.nodes)
        try:
            return orig_call(self, *args, **kwargs)
        except (fx.proxy.TraceError, RuntimeError) as e:
            if not (isinstance(e, fx.proxy.TraceError) or "symbolic tracing" in str(e)):
                raise
            added = list(graph.nodes)[mark:]
            gone = set()
            for node in reversed(added):
                gone.add(node)
                graph.erase_node(node)
            cache = item.tracer._attr_nodes
            for key in [k for k, n in cache.items() if n in gone]:
                del cache[key]
            self._autodist_leaf = True
            item.mark_control_flow(self)
            return item.tracer.create_proxy("call_module", item.path_of_module(self), args, kwargs)

    nn.Module.__init__ = tracking_init
    nn.Module.__call__ = leaf_call

    def unpatch():
        nn.Module.__init__ = orig_init
        nn.Module.__call__ = orig_call

    return unpatch
