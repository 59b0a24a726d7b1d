"""Framework patches applied while a program is captured.

Counterpart of the reference's ``autodist/patch.py:40-197`` (``PatchTensorFlow``). What needs patching in PyTorch is
much less: optimizers are captured through one wrapper on ``torch.optim.Optimizer.__init__`` (plus the ``minimize``
method), and module construction / leaf-module calls are tracked only while a scope is open. Variable-read caching and
the Keras session plumbing of the reference have no counterpart: parameters are read in place by each rank and there
is no global session object to swap.
"""
from autodist_b200 import graph_item as _gi


class PatchTorch:
    @staticmethod
    def patch_optimizers():
        """Record every optimizer constructed inside ``ad.scope()`` and give optimizers ``minimize(loss)``."""
        _gi.patch_optimizers()

    @staticmethod
    def is_patched():
        return _gi._optimizer_patched

    @staticmethod
    def suspend():
        """Context manager: objects created inside are not recorded (used by the engine for per-shard optimizers)."""
        return _gi.suspend_capture()
