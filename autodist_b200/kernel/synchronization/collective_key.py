"""Deterministic collective keys.

Every rank derives the same keys without talking to the others (capability of
``autodist/kernel/synchronization/collective_key.py:30-70``): a group key per
distinct device list (incrementing) and an instance key per variable name
(md5 folded into int32). The plan dump prints a bucket's group key and the fused engine
labels each flight's trace range with the keys of the buckets it carries
(``parallel/fused_engine.py::_on_grad_ready``), so that the same collective can be found
in every rank's trace.
"""
import hashlib
import threading

from autodist_b200.const import MAX_INT32

_lock = threading.Lock()
_singleton = None


class CollectiveKey:
    def __init__(self, group_key_start=1):
        self._group_key = group_key_start
        self._group_key_table = {}

    def generate_group_key(self, devices):
        canonical = ",".join(sorted(str(d) for d in devices))
        with _lock:
            if canonical not in self._group_key_table:
                self._group_key_table[canonical] = self._group_key
                self._group_key += 1
            return self._group_key_table[canonical]

    @staticmethod
    def generate_instance_key(var_op_name):
        return int(hashlib.md5(var_op_name.encode()).hexdigest(), 16) % MAX_INT32


def get_collective_keys():
    global _singleton
    with _lock:
        if _singleton is None:
            _singleton = CollectiveKey()
    return _singleton
