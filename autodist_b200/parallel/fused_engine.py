"""Engine selection on CUDA devices (placeholder until the fused engine lands)."""
from autodist_b200.parallel.engine import StepEngine


def make_engine(graph_item, plan, backend, device):
    return StepEngine(graph_item, plan, backend, device)
