"""Export of a trained model together with the program that trains it.

Capability parity with ``autodist/checkpoint/saved_model_builder.py:24-64``: the
builder needs this framework's ``Saver`` (so that variables are written under
their original names with partitions merged) and stores, next to the variables,
the original captured graph and the names of its placeholders / train ops so
that training can continue after reloading.

Layout: ``<export_dir>/variables/variables`` (a checkpoint of ``Saver``) and
``<export_dir>/saved_model.json`` (tags, graph text, placeholders, train ops,
strategy id).
"""
import json
import os

from autodist_b200.checkpoint.saver import Saver


class SavedModelBuilder:
    def __init__(self, export_dir):
        if os.path.exists(export_dir) and os.listdir(export_dir):
            raise AssertionError(f"export directory {export_dir} already exists and is not empty")
        self._export_dir = export_dir
        self._meta = None

    def add_meta_graph_and_variables(self, sess, tags, saver=None, signature_def_map=None, train_op=None):
        if not isinstance(saver, Saver):
            raise ValueError("add_meta_graph_and_variables needs an autodist_b200.checkpoint.saver.Saver")
        item = saver._item
        var_path = os.path.join(self._export_dir, "variables", "variables")
        saver.save(sess, var_path, write_meta_graph=False)
        from autodist_b200.autodist import get_default_autodist
        ad = get_default_autodist()
        self._meta = {
            "tags": list(tags),
            "graph": item.graph_text(),
            "placeholders": [{"name": p.name, "shape": list(p.shape), "dtype": str(p.dtype)}
                             for p in item.placeholders.values()],
            "train_ops": [op.name for op in item.train_ops] if train_op is None else [train_op.name],
            "signature_def_map": {k: str(v) for k, v in (signature_def_map or {}).items()},
            "strategy_id": ad.strategy.id if ad is not None and ad.strategy is not None else "",
            "variables": "variables/variables",
        }
        self._rank = sess.rank

    def save(self):
        if self._meta is None:
            raise RuntimeError("call add_meta_graph_and_variables first")
        if self._rank == 0:
            os.makedirs(self._export_dir, exist_ok=True)
            with open(os.path.join(self._export_dir, "saved_model.json"), "w") as f:
                json.dump(self._meta, f, indent=1)
        return self._export_dir


def load_saved_model(export_dir):
    """Plain reader: returns ``(meta dict, state dict of variables)``; needs torch only."""
    import torch
    with open(os.path.join(export_dir, "saved_model.json")) as f:
        meta = json.load(f)
    state = torch.load(os.path.join(export_dir, meta["variables"]), map_location="cpu", weights_only=False)
    return meta, state
