"""Process-wide logger (surface of the reference's ``autodist/utils/logging.py:33-146``).

One ``autodist`` logger per process writing to stderr and to
``<working dir>/logs/<timestamp>.log``; level from ``AUTODIST_MIN_LOG_LEVEL``.
"""
import logging as _logging
import os
import sys
import threading
import time

from autodist_b200 import const

_FORMAT = "[PID#%(process)d:%(asctime)s:%(filename)s#L%(lineno)d:%(levelname)s] %(message)s"
_lock = threading.Lock()
_logger = None

DEBUG, INFO, WARNING, ERROR = _logging.DEBUG, _logging.INFO, _logging.WARNING, _logging.ERROR


def get_logger():
    global _logger
    if _logger is not None:
        return _logger
    with _lock:
        if _logger is not None:
            return _logger
        lg = _logging.getLogger("autodist")
        lg.propagate = False
        level = getattr(_logging, const.ENV.AUTODIST_MIN_LOG_LEVEL.val.upper(), _logging.INFO)
        lg.setLevel(level)
        fmt = _logging.Formatter(_FORMAT)
        sh = _logging.StreamHandler(sys.stderr)
        sh.setFormatter(fmt)
        lg.addHandler(sh)
        try:
            os.makedirs(const.DEFAULT_LOG_DIR, exist_ok=True)
            fh = _logging.FileHandler(
                os.path.join(const.DEFAULT_LOG_DIR, time.strftime("%Y%m%dT%H%M%S") + f"_{os.getpid()}.log"),
                delay=True)
            fh.setFormatter(fmt)
            lg.addHandler(fh)
        except OSError:
            pass
        _logger = lg
    return _logger


def _emit(level, msg, *args):
    lg = get_logger()
    if lg.isEnabledFor(level):
        lg.log(level, msg, *args, stacklevel=3)


def debug(msg, *args):
    _emit(DEBUG, msg, *args)


def info(msg, *args):
    _emit(INFO, msg, *args)


def warning(msg, *args):
    _emit(WARNING, msg, *args)


def error(msg, *args):
    _emit(ERROR, msg, *args)


def set_verbosity(level):
    if isinstance(level, str):
        level = getattr(_logging, level.upper())
    get_logger().setLevel(level)


def get_verbosity():
    return get_logger().getEffectiveLevel()
