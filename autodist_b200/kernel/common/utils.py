"""Name helpers shared by the passes (surface of ``autodist/kernel/common/utils.py:24-99,262-272``).

The graph-surgery half of the reference's module (consumer rewiring, colocation
groups) has no counterpart: an fx graph is rewired with ``Node.replace_input_with``
and there are no colocation constraints when every rank owns one device.
"""
from collections import deque

from autodist_b200.const import AUTODIST_REPLICA_PREFIX


def get_op_name(tensor_name):
    """``"scope/w:0"`` -> ``"scope/w"`` (also strips a leading control-dependency ``^``)."""
    return tensor_name.replace("^", "").split(":")[0]


def get_index_from_tensor_name(tensor_name):
    return int(tensor_name.split(":")[1])


def replica_prefix(replica_id):
    return f"{AUTODIST_REPLICA_PREFIX}{replica_id}"


def strip_replica_prefix(name):
    for piece in name.split("/"):
        if piece.startswith(AUTODIST_REPLICA_PREFIX):
            return name[name.index(piece) + len(piece) + 1:]
    return name


def parse_name_scope(name):
    """``"a/b/c:0"`` -> ``"a/b"``; control-input marker dropped."""
    name = name.replace("^", "")
    return name.rsplit("/", 1)[0] if "/" in name else ""


def parse_optimizer_scope(update_op_name):
    """``"sgd_0/update_w"`` -> ``"sgd_0/"`` (first path element that precedes an ``update`` op)."""
    pieces = update_op_name.split("/")
    for i, piece in enumerate(pieces):
        if piece.startswith("update"):
            return "/".join(pieces[:i]) + "/" if i else ""
    return ""


def get_consumers(node):
    """fx users of a node."""
    return list(node.users)


def traverse(start, neighbors_fn, end_fn=None):
    """Breadth-first walk returning visited nodes; stops expanding where ``end_fn`` is true."""
    seen, order, queue = {start}, [], deque([start])
    while queue:
        cur = queue.popleft()
        order.append(cur)
        if end_fn is not None and end_fn(cur):
            continue
        for nxt in neighbors_fn(cur):
            if nxt not in seen:
                seen.add(nxt)
                queue.append(nxt)
    return order


def get_ancestors(nodes):
    out = set()
    for n in nodes:
        out.update(traverse(n, lambda x: x.all_input_nodes))
    return out
