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


def test_step_metrics_file(tmp_path, monkeypatch):
    import json
    import torch
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import PS
    path = tmp_path / "metrics.jsonl"
    monkeypatch.setenv("AUTODIST_METRICS_FILE", str(path))
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=PS())
    with ad.scope():
        w = torch.nn.Parameter(torch.zeros(3))
        x = ad.placeholder((None, 3), torch.float32, name="x")
        loss = ((x * w).sum(1) - 1.0).pow(2).mean()
        train_op = torch.optim.SGD([w], lr=0.1).minimize(loss)
        sess = ad.create_distributed_session()
        for _ in range(3):
            sess.run([loss, train_op], {x: torch.ones(5, 3)})
        sess.close()
    _reset_default_autodist()
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["step"] for r in rows] == [0, 1, 2]
    assert all(r["batch"] == 5 and r["host_ms"] > 0 and r["samples_per_sec"] > 0 for r in rows)
    assert rows[2]["loss"] < rows[0]["loss"]


def test_function_with_keyword_arguments_and_second_function_refused():
    import numpy as np
    import torch
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import AllReduce
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=AllReduce())
    with ad.scope():
        w = torch.nn.Parameter(torch.zeros(3))
        opt = torch.optim.SGD([w], lr=0.1)

        @ad.function
        def step(x, y=None):
            loss = ((x * w).sum(1) - y).pow(2).mean()
            return loss, opt.minimize(loss)

        x, y = np.ones((4, 3), np.float32), np.ones(4, np.float32)
        first, _ = step(x, y=y)
        second, _ = step(x[:2], y=y[:2])                  # the batch dimension is free
        assert float(second) < float(first)

        @ad.function
        def other(x):
            return (x * w).sum()

        with pytest.raises(NotImplementedError):
            other(x)
    _reset_default_autodist()
