"""Named ranges for timeline tools, off by default.

``AUTODIST_NVTX=1`` wraps every training call (``step <n>``) and every gradient flight
(``flight [lo, hi)``) in an NVTX range so that they show up as labelled spans on the CPU
thread of a timeline capture; without the variable (or without CUDA) ``annotate`` costs one
dictionary lookup.
"""
import contextlib
import os

import torch


def enabled():
    return os.environ.get("AUTODIST_NVTX", "0") not in ("0", "", "False", "false") and torch.cuda.is_available()


@contextlib.contextmanager
def annotate(name):
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
