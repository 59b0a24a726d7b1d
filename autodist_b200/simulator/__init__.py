"""Strategy cost model and ranking (the reference ships only the dataset description of its simulator,
``autodist/simulator/dataset/README.md``; the model here is re-fit to NVLink 5 / NVSwitch)."""
from autodist_b200.simulator.cost_model import LinkModel, NVSwitchCostModel  # noqa: F401
from autodist_b200.simulator.simulator import Simulator, rank_strategies  # noqa: F401
