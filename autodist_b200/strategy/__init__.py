"""Strategy builders (same eight names as the reference's ``autodist/strategy/__init__.py:20-27``)."""
from autodist_b200.strategy.base import Strategy, StrategyBuilder, StrategyCompiler  # noqa: F401
from autodist_b200.strategy.ps_strategy import PS, PSLoadBalancing  # noqa: F401
from autodist_b200.strategy.partitioned_ps_strategy import PartitionedPS, UnevenPartitionedPS  # noqa: F401
from autodist_b200.strategy.all_reduce_strategy import AllReduce, PartitionedAR, RandomAxisPartitionAR  # noqa: F401
from autodist_b200.strategy.parallax_strategy import Parallax  # noqa: F401
from autodist_b200.strategy.auto_strategy import AutoStrategy  # noqa: F401
