"""Python face of the hand-written sm_100a kernels.

``ext()`` returns the compiled extension module. On a machine with a CUDA device
a missing or stale extension is an error (no silent PyTorch fallback); without a
device ``ext()`` returns ``None`` and only the host-side logic is usable.
"""
import importlib.util
import os
import sys

import torch

from autodist_b200.ops import build as _build

_EXT = None
_TRIED = False
launch_count = 0      # kernels launched through the extension by this process (a graph replay re-launches its capture)


class _Counting:
    """Thin proxy over the extension module that counts kernel-launching calls."""
    _NO_LAUNCH = {"ln_bwd_blocks", "ln_bwd_part_floats", "colsum_parts", "MAX_COMM_BLOCKS"}
    _MULTI = {"ln_bwd": 2, "keyed_colsum": 2, "bn_fwd": 3, "bn_bwd": 3}

    def __init__(self, mod):
        self._mod = mod
        for name in dir(mod):
            if name.startswith("_"):
                continue
            attr = getattr(mod, name)
            if callable(attr) and name not in self._NO_LAUNCH:
                setattr(self, name, self._wrap(attr, self._MULTI.get(name, 1)))
            else:
                setattr(self, name, attr)

    @staticmethod
    def _wrap(fn, n):
        def call(*args):
            global launch_count
            launch_count += n
            return fn(*args)
        return call


def ext(required=None):
    global _EXT, _TRIED
    if _EXT is not None:
        return _EXT
    if required is None:
        required = torch.cuda.is_available()
    if not _TRIED or required:
        _TRIED = True
        path = _build.so_path()
        stale = os.path.exists(path) and not _build.is_current()
        if (not os.path.exists(path) or stale) and required:
            path = _build.build()              # rebuilds when the sources changed since the shared object was made
        elif stale:
            raise RuntimeError("the sm_100a extension is older than its sources: run `python -m autodist_b200.ops.build`")
        if os.path.exists(path):
            spec = importlib.util.spec_from_file_location(_build.NAME, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.modules[_build.NAME] = mod
            _EXT = _Counting(mod)
    if _EXT is None and required:
        raise RuntimeError("the sm_100a extension is not built: run `python -m autodist_b200.ops.build`")
    return _EXT
