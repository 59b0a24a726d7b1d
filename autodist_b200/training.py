"""``compile`` / ``fit`` / ``evaluate`` / ``predict`` on top of a distributed session.

The reference makes Keras' ``model.compile / fit / evaluate`` run on its session by patching Keras internals
(``autodist/patch.py:96-197``; exercised by ``tests/integration/cases/c7.py:12-24``). PyTorch has no such training
loop to patch, so this module provides one with the same surface: the model is traced once with batch-split
placeholders, the optimizer is captured like any other, and every batch is one ``session.run``.

    ad = AutoDist(resource_spec_file, AllReduce())
    model = Model(ad, lambda: MyNet())                     # the module is built inside ad.scope()
    model.compile(optimizer=lambda ps: torch.optim.SGD(ps, lr=0.1), loss=torch.nn.functional.cross_entropy,
                  metrics={"accuracy": lambda out, y: (out.argmax(1) == y).float().mean()})
    history = model.fit(x, y, batch_size=64, epochs=2)
    print(model.evaluate(x, y, batch_size=64))

Every process runs the same script and feeds its node's batches (``batch_size`` per replica times the replicas of
the node), as the reference's workers do; metrics are those of the feeding node.
"""
from typing import Callable, Dict, Optional

import numpy as np
import torch
from torch import nn


def _as_tuple(x):
    return tuple(x) if isinstance(x, (list, tuple)) else (x,)


def _to_tensor(a):
    return a if torch.is_tensor(a) else torch.as_tensor(np.asarray(a))


class History:
    """``history[name]`` is the list of per-epoch means, as in ``keras.callbacks.History.history``."""

    def __init__(self):
        self.history: Dict[str, list] = {}
        self.epoch = []

    def record(self, epoch, values):
        self.epoch.append(epoch)
        for k, v in values.items():
            self.history.setdefault(k, []).append(v)


class Model:
    def __init__(self, autodist, module_fn: Callable[[], nn.Module]):
        """``module_fn`` builds the ``nn.Module``; it is called inside ``autodist.scope()`` so that the module's
        parameters become the variables of the captured graph."""
        self._ad = autodist
        self._module_fn = module_fn
        self._compiled = None
        self._built = None
        self.module: Optional[nn.Module] = None

    # ------------------------------------------------------------------ compile
    def compile(self, optimizer, loss, metrics: Optional[Dict[str, Callable]] = None, clip_global_norm=None):
        """``optimizer``: ``callable(parameters) -> torch.optim.Optimizer`` (or an optimizer class, constructed with
        its defaults); ``loss``: ``callable(outputs, targets) -> scalar``; ``metrics``: name -> ``callable(outputs,
        targets) -> scalar``; ``clip_global_norm``: joint gradient-norm bound over all parameters."""
        if isinstance(optimizer, torch.optim.Optimizer):
            raise TypeError("pass a factory (parameters -> optimizer) or an optimizer class: the optimizer has to be "
                            "constructed inside the scope to be captured")
        self._compiled = (optimizer, loss, dict(metrics or {}), clip_global_norm)
        return self

    def _build(self, x, y):
        if self._built is not None:
            return self._built
        if self._compiled is None:
            raise RuntimeError("call compile() before fit / evaluate")
        opt_fn, loss_fn, metrics, clip = self._compiled
        ad = self._ad
        xs = _as_tuple(x)
        with ad.scope():
            self.module = self._module_fn()
            x_ph = [ad.placeholder((None,) + tuple(t.shape[1:]), t.dtype, name=f"x{i}") for i, t in enumerate(xs)]
            y_ph = ad.placeholder((None,) + tuple(y.shape[1:]), y.dtype, name="y") if y is not None else None
            out = self.module(*x_ph)
            fetch = {"outputs": out}
            train_op = None
            if y_ph is not None:
                loss = loss_fn(out, y_ph)
                fetch["loss"] = loss
                for name, fn in metrics.items():
                    fetch[name] = fn(out, y_ph)
                params = [p for p in self.module.parameters() if p.requires_grad]
                opt = opt_fn(params)
                train_op = opt.minimize(loss, clip_global_norm=(clip, params) if clip else None)
                self.optimizer = opt
            sess = ad.create_distributed_session()
        self._built = (sess, x_ph, y_ph, fetch, train_op)
        return self._built

    @property
    def session(self):
        return self._built[0] if self._built else None

    # ------------------------------------------------------------------ loops
    def _node_batch(self, batch_size):
        return batch_size * max(1, getattr(self._built[0].remapper, "num_local_replicas", 1)) if self._built else batch_size

    @staticmethod
    def _batches(n, node_batch, steps, order):
        count = 0
        for lo in range(0, n, node_batch):
            if steps is not None and count >= steps:
                return
            yield order[lo:lo + node_batch]
            count += 1

    def fit(self, x, y, batch_size=32, epochs=1, steps_per_epoch=None, shuffle=False, seed=0, verbose=0, callbacks=()):
        xs = tuple(_to_tensor(a) for a in _as_tuple(x))
        y = _to_tensor(y)
        sess, x_ph, y_ph, fetch, train_op = self._build(xs, y)
        names = [k for k in fetch if k != "outputs"]
        history = History()
        n = xs[0].shape[0]
        node_batch = self._node_batch(batch_size)
        gen = torch.Generator().manual_seed(seed)
        for epoch in range(epochs):
            order = torch.randperm(n, generator=gen) if shuffle else torch.arange(n)
            sums, seen = {k: 0.0 for k in names}, 0
            for idx in self._batches(n, node_batch, steps_per_epoch, order):
                feed = {ph: t[idx] for ph, t in zip(x_ph, xs)}
                feed[y_ph] = y[idx]
                vals = sess.run([fetch[k] for k in names] + [train_op], feed)
                for k, v in zip(names, vals):
                    sums[k] += float(np.mean(v)) * len(idx)
                seen += len(idx)
            means = {k: s / max(seen, 1) for k, s in sums.items()}
            history.record(epoch, means)
            for cb in callbacks:
                cb(epoch, means)
            if verbose and sess.rank == 0:
                print(f"epoch {epoch + 1}/{epochs} " + " ".join(f"{k} {v:.4f}" for k, v in means.items()), flush=True)
        return history

    def evaluate(self, x, y, batch_size=32, steps=None):
        """Mean loss and metrics over ``(x, y)`` without touching the parameters."""
        xs = tuple(_to_tensor(a) for a in _as_tuple(x))
        y = _to_tensor(y)
        sess, x_ph, y_ph, fetch, _ = self._build(xs, y)
        names = [k for k in fetch if k != "outputs"]
        n = xs[0].shape[0]
        sums, seen = {k: 0.0 for k in names}, 0
        for idx in self._batches(n, self._node_batch(batch_size), steps, torch.arange(n)):
            feed = {ph: t[idx] for ph, t in zip(x_ph, xs)}
            feed[y_ph] = y[idx]
            vals = sess.run([fetch[k] for k in names], feed)
            for k, v in zip(names, vals):
                sums[k] += float(np.mean(v)) * len(idx)
            seen += len(idx)
        return {k: s / max(seen, 1) for k, s in sums.items()}

    def predict(self, x, batch_size=32):
        xs = tuple(_to_tensor(a) for a in _as_tuple(x))
        if self._built is None:
            raise RuntimeError("predict() needs a built model: call fit() or evaluate() first")
        sess, x_ph, _, fetch, _ = self._built
        n = xs[0].shape[0]
        outs = []
        for idx in self._batches(n, self._node_batch(batch_size), None, torch.arange(n)):
            outs.append(np.asarray(sess.run(fetch["outputs"], {ph: t[idx] for ph, t in zip(x_ph, xs)})))
        return np.concatenate(outs, 0)
