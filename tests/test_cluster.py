"""Cluster description, device resolution, remote command construction (dry run) and the coordinator's worker environment."""
import os

import numpy as np
import torch

from autodist_b200.cluster import SSHCluster
from autodist_b200.coordinator import Coordinator
from autodist_b200.kernel.device.resolver import DeviceResolver
from autodist_b200.kernel.replicator import Replicator
from autodist_b200.remapper import _chunk_bounds
from autodist_b200.resource_spec import ResourceSpec, SSHConfig
from autodist_b200.strategy.base import Strategy

SPECS = os.path.join(os.path.dirname(__file__), "resource_specs")


def test_cluster_spec_and_ranks():
    c = SSHCluster(ResourceSpec(os.path.join(SPECS, "r4.yml")))      # 2 GPUs on .57 (chief), 1 GPU on .146
    assert c.nodes == ["10.20.41.146", "10.20.41.57"]
    assert [a.rsplit(":", 1)[0] for a in c.cluster_spec["worker"]] == c.nodes
    assert c.world_size == 3 and c.chief_rank == 1
    assert c.ranks_of_node("10.20.41.57") == [1, 2] and c.local_rank_of(2) == 1
    assert c.is_chief("10.20.41.57") and not c.is_chief("10.20.41.146")
    assert c.get_address_from_task("worker", 0) == "10.20.41.146"


def test_device_resolver_and_replicator():
    c = SSHCluster(ResourceSpec(os.path.join(SPECS, "r1.yml")))
    r = DeviceResolver(c)
    assert r.resolve_to_device_str("10.20.41.57:GPU:1") == "/job:worker/task:1/device:GPU:1/rank:3"
    cpu = r.resolve_to_device_str("10.20.41.146:CPU:0")               # a node's CPU -> its first replica's rank
    assert cpu == "/job:worker/task:0/device:CPU:0/rank:0" and DeviceResolver.rank_of(cpu) == 0
    replicas = r.resolve_to_device_str(c.replica_devices)
    info = Replicator.apply(replicas, 2)
    assert info.world_size == 4 and info.local_ranks == [2, 3] and info.local_replica_index == 0 and info.num_workers == 2


def test_remote_command_dry_run(monkeypatch):
    monkeypatch.setenv("AUTODIST_DEBUG_REMOTE", "True")
    rs = ResourceSpec(os.path.join(SPECS, "r4.yml"))
    c = SSHCluster(rs)
    c._ssh_conf = {"10.20.41.146": SSHConfig(username="root", port=12345, python_venv="source /opt/venv/bin/activate",
                                             key_file="/home/u/.ssh/id_rsa", env={"LD_LIBRARY_PATH": "/usr/local/cuda/lib64"})}
    cmd = c.remote_command(["python", "/abs/train.py", "--x", "1"], "10.20.41.146", {"AUTODIST_WORKER": "10.20.41.146:GPU:0"})
    joined = " ".join(cmd)
    assert cmd[0] == "ssh" and "-p 12345" in joined and "-i /home/u/.ssh/id_rsa" in joined and "root@10.20.41.146" in joined
    assert "source /opt/venv/bin/activate" in joined and "AUTODIST_WORKER=10.20.41.146:GPU:0" in joined
    assert "LD_LIBRARY_PATH=/usr/local/cuda/lib64" in joined and "/abs/train.py" in joined
    assert c.remote_exec(["true"], "10.20.41.146") is None          # dry run: nothing is started
    assert c.remote_copy("/tmp/a", "/tmp/a", "10.20.41.146") is None


def test_coordinator_worker_environment():
    c = SSHCluster(ResourceSpec(os.path.join(SPECS, "r0.yml")))
    s = Strategy()
    env = Coordinator(s, c)._worker_env(1)
    assert env["AUTODIST_WORKER"] == "localhost:GPU:1" and env["AUTODIST_STRATEGY_ID"] == s.id
    assert env["RANK"] == "1" and env["WORLD_SIZE"] == "2" and env["LOCAL_RANK"] == "1" and env["MASTER_ADDR"]


def test_feed_chunks_follow_array_split():
    for n in (1, 7, 8, 31, 64):
        for k in (1, 2, 3, 8):
            ref = np.array_split(np.arange(n), k)
            for i in range(k):
                lo, hi = _chunk_bounds(n, k, i)
                assert list(range(lo, hi)) == ref[i].tolist()


def test_patch_and_starter_import():
    from autodist_b200.patch import PatchTorch
    from autodist_b200.utils import server_starter
    PatchTorch.patch_optimizers()
    assert PatchTorch.is_patched() and hasattr(torch.optim.SGD, "minimize")
    assert callable(server_starter.main)
