"""Stage dumps of the transformation (text and DOT files instead of TensorBoard events).

Reference: ``autodist/utils/visualization_util.py:24-36`` writes the graph after
each transformer stage under ``<working dir>/graphs/<stage>``; the same stage
names are used here and the payload is the fx graph / plan description. Dumps are
written when ``AUTODIST_DUMP_GRAPHS=1``; the DOT files need no renderer to be read
and load into any Graphviz viewer.
"""
import os

from autodist_b200 import const


def enabled():
    return os.environ.get("AUTODIST_DUMP_GRAPHS", "0") not in ("0", "", "False", "false")


def log_graph(text, name):
    if not enabled():
        return None
    os.makedirs(const.DEFAULT_GRAPH_DIR, exist_ok=True)
    path = os.path.join(const.DEFAULT_GRAPH_DIR, f"{name}.{os.getpid()}.txt")
    with open(path, "w") as f:
        f.write(text if isinstance(text, str) else str(text))
    return path


def fx_graph_to_dot(graph, name="captured"):
    """DOT text of a ``torch.fx.Graph``: one node per fx node (placeholders as boxes, parameters as ellipses with a
    double border, outputs as octagons), one edge per data dependency."""
    shapes = {"placeholder": "box", "get_attr": "doublecircle", "output": "octagon"}
    lines = [f'digraph "{name}" {{', "  rankdir=TB;", '  node [fontname="monospace", fontsize=10];']
    for node in graph.nodes:
        target = node.target if isinstance(node.target, str) else getattr(node.target, "__name__", str(node.target))
        label = f"{node.name}\\n{node.op}: {target}".replace('"', "'")
        lines.append(f'  "{node.name}" [label="{label}", shape={shapes.get(node.op, "ellipse")}];')
    for node in graph.nodes:
        for src in node.all_input_nodes:
            lines.append(f'  "{src.name}" -> "{node.name}";')
    lines.append("}")
    return "\n".join(lines) + "\n"


def log_fx_graph(graph, name):
    """Write ``<name>.<pid>.dot`` beside the text dumps; returns the path or ``None`` when dumps are off."""
    if not enabled():
        return None
    os.makedirs(const.DEFAULT_GRAPH_DIR, exist_ok=True)
    path = os.path.join(const.DEFAULT_GRAPH_DIR, f"{name}.{os.getpid()}.dot")
    with open(path, "w") as f:
        f.write(fx_graph_to_dot(graph, name))
    return path
