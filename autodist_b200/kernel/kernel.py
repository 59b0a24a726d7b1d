"""Pass protocol: ``SomePass.apply(*args)`` constructs the pass and runs it.

Same calling convention as the reference's ``autodist/kernel/kernel.py:19-35``;
direct construction is reserved to ``apply`` so that a pass is never half-run.
"""
from abc import ABC, abstractmethod

_TOKEN = object()


class Kernel(ABC):
    def __init__(self, key=None):
        if key is not _TOKEN:
            raise ValueError("use %s.apply(...) instead of constructing the pass" % type(self).__name__)

    @classmethod
    def apply(cls, *args, **kwargs):
        obj = cls(_TOKEN, *args, **kwargs)
        return obj._apply()

    @abstractmethod
    def _apply(self):
        raise NotImplementedError
