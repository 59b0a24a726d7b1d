"""autodist_b200: a Blackwell-native auto-distribution training engine for PyTorch.

Same public surface as petuum/autodist (``autodist/__init__.py``, ``autodist/autodist.py``):
``AutoDist``, strategy builders under ``autodist_b200.strategy``, the checkpoint
``Saver`` under ``autodist_b200.checkpoint.saver``.
"""
from autodist_b200.const import ENV  # noqa: F401
from autodist_b200.utils import logging as _logging

_logging.get_logger()

from autodist_b200.autodist import AutoDist, IS_AUTODIST_CHIEF, IS_AUTODIST_WORKER  # noqa: E402,F401
from autodist_b200.autodist import get_default_autodist  # noqa: E402,F401
from autodist_b200.graph_item import graph_op  # noqa: E402,F401
from autodist_b200 import strategy  # noqa: E402,F401

__version__ = "0.1.0"
