"""compile / fit / evaluate / predict facade (CPU, single replica and two gloo ranks)."""
import numpy as np
import pytest
import torch
from torch import nn

from autodist_b200 import AutoDist
from autodist_b200.autodist import _reset_default_autodist
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200 import strategy as S
from autodist_b200.training import Model


def _data(n=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 6, generator=g)
    w = torch.randn(6, 3, generator=g)
    return x, (x @ w).argmax(1)


@pytest.mark.parametrize("builder", [S.PSLoadBalancing, S.AllReduce, S.PartitionedPS])
def test_fit_evaluate_predict(builder):
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=builder())
    x, y = _data()
    torch.manual_seed(1)
    model = Model(ad, lambda: nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 3)))
    with pytest.raises(TypeError):
        model.compile(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1), nn.functional.cross_entropy)
    model.compile(lambda ps: torch.optim.SGD(ps, lr=0.3), nn.functional.cross_entropy,
                  metrics={"accuracy": lambda out, t: (out.argmax(1) == t).float().mean()})
    seen = []
    hist = model.fit(x, y, batch_size=16, epochs=6, shuffle=True, callbacks=[lambda e, m: seen.append(e)])
    assert seen == list(range(6)) and hist.epoch == seen
    assert hist.history["loss"][-1] < hist.history["loss"][0]
    ev = model.evaluate(x, y, batch_size=32)
    assert set(ev) == {"loss", "accuracy"} and ev["accuracy"] > 0.5
    again = model.evaluate(x, y, batch_size=32)
    assert again == ev                                   # evaluation leaves the parameters alone
    pred = model.predict(x, batch_size=40)
    assert pred.shape == (96, 3)
    assert np.mean(pred.argmax(1) == y.numpy()) == pytest.approx(ev["accuracy"], abs=1e-6)
    model.session.close()
    _reset_default_autodist()


def test_fit_matches_plain_pytorch():
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=S.AllReduce())
    x, y = _data(32, seed=3)
    torch.manual_seed(5)
    ref = nn.Sequential(nn.Linear(6, 8), nn.ReLU(), nn.Linear(8, 3))
    state = {k: v.clone() for k, v in ref.state_dict().items()}

    def build():
        m = nn.Sequential(nn.Linear(6, 8), nn.ReLU(), nn.Linear(8, 3))
        m.load_state_dict(state)
        return m

    model = Model(ad, build).compile(lambda ps: torch.optim.SGD(ps, lr=0.1, momentum=0.9), nn.functional.cross_entropy)
    hist = model.fit(x, y, batch_size=8, epochs=2, steps_per_epoch=3)
    opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    losses = []
    for _ in range(2):
        tot = 0.0
        for lo in range(0, 24, 8):
            opt.zero_grad()
            loss = nn.functional.cross_entropy(ref(x[lo:lo + 8]), y[lo:lo + 8])
            loss.backward()
            opt.step()
            tot += float(loss.detach()) * 8
        losses.append(tot / 24)
    assert hist.history["loss"] == pytest.approx(losses, rel=1e-5)
    got = model.predict(x)
    torch.testing.assert_close(torch.as_tensor(got), ref(x).detach(), rtol=1e-5, atol=1e-6)
    model.session.close()
    _reset_default_autodist()


@pytest.mark.integration
def test_fit_route_of_the_example_on_two_self_launched_ranks():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "AUTODIST_WORKER",
                                                            "AUTODIST_STRATEGY_ID")}
    env["AUTODIST_MIN_LOG_LEVEL"] = "ERROR"
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "image_classifier.py"), "--fit"], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "epoch 3/3" in r.stdout and "evaluate:" in r.stdout


@pytest.mark.integration
def test_record_feeder_route_of_the_example_on_two_self_launched_ranks():
    """Batches from the native feeder, each step prefetching the next batch, on two CPU replicas started by the chief."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "AUTODIST_WORKER",
                                                            "AUTODIST_STRATEGY_ID")}
    env["AUTODIST_MIN_LOG_LEVEL"] = "ERROR"
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "image_classifier.py"), "--feeder"], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    losses = [float(l.split()[-1]) for l in r.stdout.splitlines() if l.startswith("step ")]
    assert len(losses) == 5 and losses[-1] < losses[0], r.stdout          # 20 steps, printed every fourth
