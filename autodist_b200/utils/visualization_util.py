"""Stage dumps of the transformation (text files instead of TensorBoard events).

Reference: ``autodist/utils/visualization_util.py:24-36`` writes the graph after
each transformer stage under ``<working dir>/graphs/<stage>``; the same stage
names are used here and the payload is the fx graph / plan description.
"""
import os

from autodist_b200 import const

_enabled = os.environ.get("AUTODIST_DUMP_GRAPHS", "0") not in ("0", "", "False")


def log_graph(text, name):
    if not _enabled:
        return None
    os.makedirs(const.DEFAULT_GRAPH_DIR, exist_ok=True)
    path = os.path.join(const.DEFAULT_GRAPH_DIR, f"{name}.{os.getpid()}.txt")
    with open(path, "w") as f:
        f.write(text if isinstance(text, str) else str(text))
    return path
