"""Checkpoints that a plain single-device PyTorch program can read.

Capability parity with ``autodist/checkpoint/saver.py:27-133``: the saver must
exist before the distributed session is created, and what it writes uses the
*original* single-device variable names and full shapes - shards of a
partitioned variable (and of its optimizer slots) are merged back at their
offsets (the reference does this with ``SaveSliceInfo``,
``autodist/kernel/partitioner.py:292-347``). So

    state = torch.load("model-100")
    model.load_state_dict(state["variables"])

works without importing this framework, and a checkpoint written under one
strategy restores under any other (restore re-shards by the current plan).

Files: ``<path>-<step>`` (``torch.save`` of ``{"variables", "slots",
"global_step", "slices"}``), ``<path>-<step>.index`` (JSON: names, shapes, how
each variable was sharded when saved) and ``checkpoint`` in the same directory
(latest + kept paths), with ``max_to_keep`` rotation.
"""
import json
import os

import torch

from autodist_b200 import graph_item as _gi
from autodist_b200.utils import logging


def _strip(name):
    return name[:-2] if name.endswith(":0") else name


class Saver:
    def __init__(self, var_list=None, max_to_keep=5, save_relative_paths=True, name=None):
        item = _gi.get_default_graph_item()
        if item is None:
            from autodist_b200.autodist import get_default_autodist
            ad = get_default_autodist()
            item = ad.graph_item if ad is not None else None
        if item is None:
            raise RuntimeError("create the Saver inside ad.scope()")
        from autodist_b200.autodist import get_default_autodist
        ad = get_default_autodist()
        if ad is not None and ad._session is not None:
            raise RuntimeError("Saver must be created before create_distributed_session()")
        self._item = item
        self._var_list = None if var_list is None else [
            v if isinstance(v, str) else item.name_of_parameter(v) for v in var_list]
        self._max_to_keep = max_to_keep
        self._relative = save_relative_paths
        self._kept = []
        self.name = name or f"save_{len(item.savers)}"
        item.update_savers(self)

    def saver_def(self):
        return {"name": self.name, "max_to_keep": self._max_to_keep, "var_list": self._var_list}

    # ------------------------------------------------------------------ save
    def _collect(self, engine):
        variables, slices = {}, {}
        names = self._var_list or [n for n, _ in self._item.named_parameters()]
        for name in names:
            variables[_strip(name)] = engine.variable_value(name).detach().cpu().clone()
            sp = engine.plan.shard_plans.get(name)
            if sp is not None:
                slices[_strip(name)] = [list(sp.save_slice_info(i)[2:]) for i in range(sp.num_shards)]
        if self._var_list is None:
            for bname, b in self._item.named_buffers():
                variables[bname] = b.detach().cpu().clone()
        slots = {k: v.detach().cpu() for k, v in engine.optimizer_slots().items()}
        return variables, slots, slices

    def save(self, sess, save_path, global_step=None, write_meta_graph=True):
        engine = sess.engine
        variables, slots, slices = self._collect(engine)   # collective: every rank takes part
        path = save_path if global_step is None else f"{save_path}-{int(global_step)}"
        if engine.rank != 0:
            return path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        tmp = path + ".tmp"
        torch.save({"variables": variables, "slots": slots, "slices": slices,
                    "global_step": engine.global_step if global_step is None else int(global_step)}, tmp)
        os.replace(tmp, path)
        with open(path + ".index", "w") as f:
            json.dump({"variables": {k: list(v.shape) for k, v in variables.items()},
                       "slots": {k: list(v.shape) for k, v in slots.items()}, "slices": slices}, f)
        if write_meta_graph:
            with open(path + ".meta", "w") as f:
                f.write(self._item.graph_text())
        self._rotate(path)
        logging.debug("saved checkpoint %s", path)
        return path

    def _rotate(self, path):
        if path in self._kept:
            self._kept.remove(path)
        self._kept.append(path)
        while self._max_to_keep and len(self._kept) > self._max_to_keep:
            old = self._kept.pop(0)
            for suffix in ("", ".index", ".meta"):
                try:
                    os.remove(old + suffix)
                except FileNotFoundError:
                    pass
        directory = os.path.dirname(os.path.abspath(path))
        rel = (lambda p: os.path.basename(p)) if self._relative else (lambda p: p)
        with open(os.path.join(directory, "checkpoint"), "w") as f:
            json.dump({"model_checkpoint_path": rel(path),
                       "all_model_checkpoint_paths": [rel(p) for p in self._kept]}, f)

    # ------------------------------------------------------------------ restore
    def restore(self, sess, save_path):
        engine = sess.engine
        state = torch.load(save_path, map_location="cpu", weights_only=False)
        params = dict(self._item.named_parameters())
        with torch.no_grad():
            for name, p in params.items():
                key = _strip(name)
                if key in state["variables"] and (self._var_list is None or name in self._var_list):
                    p.data.copy_(state["variables"][key].to(p.device, p.dtype))
            for bname, b in self._item.named_buffers():
                if bname in state["variables"]:
                    b.data.copy_(state["variables"][bname].to(b.device, b.dtype))
        engine.global_step = int(state.get("global_step", 0))
        engine.load_optimizer_slots(state.get("slots", {}), default_step=engine.global_step)
        if hasattr(engine, "after_restore"):
            engine.after_restore()
        return state


def latest_checkpoint(checkpoint_dir):
    index = os.path.join(checkpoint_dir, "checkpoint")
    if not os.path.exists(index):
        return None
    with open(index) as f:
        rec = json.load(f)
    p = rec["model_checkpoint_path"]
    return p if os.path.isabs(p) else os.path.join(checkpoint_dir, p)
