"""Resource spec and device spec parsing (mirrors the intent of the reference's
``tests/test_resource_spec.py`` and ``tests/test_device_spec.py``)."""
import os

import pytest

from autodist_b200.resource_spec import Connectivity, DeviceSpec, DeviceType, ResourceSpec

SPECS = os.path.join(os.path.dirname(__file__), "resource_specs")


@pytest.mark.parametrize("i", range(10))
def test_all_specs_parse(i):
    rs = ResourceSpec(os.path.join(SPECS, f"r{i}.yml"))
    assert rs.chief
    assert len(rs.replica_devices) >= 1
    for node in rs.nodes:
        assert rs.network_bandwidth[node] >= 1


def test_counts():
    r0 = ResourceSpec(os.path.join(SPECS, "r0.yml"))
    assert (r0.num_gpus, r0.num_cpus) == (2, 1)
    r5 = ResourceSpec(os.path.join(SPECS, "r5.yml"))
    assert (r5.num_gpus, r5.num_cpus) == (0, 2)
    r4 = ResourceSpec(os.path.join(SPECS, "r4.yml"))
    assert r4.num_gpus == 3 and len(r4.nodes) == 2
    assert r4.network_bandwidth == {"10.20.41.57": 100, "10.20.41.146": 50}


def test_bandwidth_default():
    r0 = ResourceSpec(os.path.join(SPECS, "r0.yml"))
    assert r0.network_bandwidth["localhost"] == 1


def test_replica_rule_and_rank_order():
    r1 = ResourceSpec(os.path.join(SPECS, "r1.yml"))
    # sorted node addresses (string order), device index within a node
    assert r1.replica_devices == ["10.20.41.146:GPU:0", "10.20.41.146:GPU:1", "10.20.41.57:GPU:0", "10.20.41.57:GPU:1"]
    r9 = ResourceSpec(os.path.join(SPECS, "r9.yml"))
    assert r9.replica_devices == ["10.20.41.146:CPU:0", "10.20.41.57:CPU:0", "10.20.41.57:CPU:1"]


def test_errors(tmp_path):
    p = tmp_path / "bad.yml"
    p.write_text("nodes:\n  - address: localhost\n    gpus: [0]\n  - address: 10.0.0.2\n    gpus: [0]\n")
    with pytest.raises(ValueError):
        ResourceSpec(str(p))     # loopback with several nodes
    p.write_text("nodes:\n  - address: 10.0.0.1\n    gpus: [0]\n    chief: true\n  - address: 10.0.0.2\n    gpus: [0]\n")
    with pytest.raises(ValueError):
        ResourceSpec(str(p))     # non-chief without ssh_config
    p.write_text("nodes:\n  - address: 10.0.0.1\n    gpus: [0]\n    ssh_config: c\n  - address: 10.0.0.2\n"
                 "    gpus: [0]\n    ssh_config: c\nssh:\n  c:\n    username: u\n")
    with pytest.raises(ValueError):
        ResourceSpec(str(p))     # nobody is chief


def test_device_spec_round_trip():
    for name in ("10.0.0.1:GPU:3", "localhost:CPU:0", "host-a:CPU:2"):
        assert DeviceSpec.from_string(name).name_string() == name
    d = DeviceSpec.from_string("10.0.0.1:GPU:3")
    assert d.device_type is DeviceType.GPU and d.device_index == 3 and d.host_device.name_string() == "10.0.0.1:CPU:0"
    assert d.connectivity_with(DeviceSpec.from_string("10.0.0.1:GPU:1")) is Connectivity.NVSWITCH
    assert d.connectivity_with(DeviceSpec.from_string("10.0.0.2:GPU:1")) is Connectivity.ETHERNET


def test_ssh_config():
    r4 = ResourceSpec(os.path.join(SPECS, "r4.yml"))
    assert r4.ssh_group["10.20.41.146"] == "conf"
    # the map is only built on the chief's own machine; parse the section directly to check the fields
    from autodist_b200.resource_spec import SSHConfig
    conf = SSHConfig.from_info({"username": "root", "port": 12345, "shared_envs": {"A": 1}})
    assert conf.port == 12345 and conf.env["A"] == "1" and conf.username == "root"
