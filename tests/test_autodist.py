import pytest

from autodist_b200 import AutoDist
from autodist_b200.autodist import _reset_default_autodist
from autodist_b200.resource_spec import ResourceSpec


def test_single_instance_per_process():
    _reset_default_autodist()
    AutoDist(resource_spec=ResourceSpec.local(num_cpus=1))
    with pytest.raises(NotImplementedError):
        AutoDist(resource_spec=ResourceSpec.local(num_cpus=1))
    _reset_default_autodist()
