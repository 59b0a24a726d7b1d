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


def test_step_deadline_watchdog_reports_a_slow_step(monkeypatch, capfd):
    import time
    import torch
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import PS

    class Slow(torch.nn.Module):
        _autodist_leaf = True                        # runs at step time, not at trace time

        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(2))
            self.delay = 0.0

        def forward(self, x):
            time.sleep(self.delay)
            return ((x * self.w).sum(1) - 1.0).pow(2).mean()

    monkeypatch.setenv("AUTODIST_STEP_TIMEOUT", "1.0")
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=PS())
    with ad.scope():
        m = Slow()
        x = ad.placeholder((None, 2), torch.float32, name="x")
        loss = m(x)
        train_op = torch.optim.SGD(m.parameters(), lr=0.1).minimize(loss)
        sess = ad.create_distributed_session()
        feed = {x: torch.ones(3, 2)}
        sess.run([loss, train_op], feed)             # warm-up (tracing, first launch); may or may not be slow
        base = sess._watchdog.fired
        m.delay = 3.0
        sess.run([loss, train_op], feed)             # the step still completes; the watchdog only reports
        assert sess._watchdog.fired >= base + 1
        sess.close()
    _reset_default_autodist()
    err = capfd.readouterr().err
    assert "most recent call first" in err and "time.sleep" not in err.split("most recent call first")[0]
    assert "forward" in err                            # the stack dump shows where the slow step was


def test_step_deadline_abort_ends_the_process_with_code_70(tmp_path):
    import os
    import subprocess
    import sys
    script = tmp_path / "slow.py"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script.write_text(f'''
import sys, time
sys.path.insert(0, {root!r})
import torch
from autodist_b200 import AutoDist
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200.strategy import PS

class Stuck(torch.nn.Module):
    _autodist_leaf = True
    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.zeros(2))
    def forward(self, x):
        time.sleep(30)                                # stands for a rank that never comes back from a collective
        return (x * self.w).sum()

ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=PS())
with ad.scope():
    m = Stuck()
    x = ad.placeholder((None, 2), torch.float32, name="x")
    loss = m(x)
    op = torch.optim.SGD(m.parameters(), lr=0.1).minimize(loss)
    sess = ad.create_distributed_session()
    sess.run([loss, op], {{x: torch.ones(1, 2)}})
print("not reached")
''')
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE")}
    env.update(AUTODIST_STEP_TIMEOUT="0.5", AUTODIST_STEP_TIMEOUT_ACTION="abort", AUTODIST_MIN_LOG_LEVEL="ERROR")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 70, r.stderr[-2000:]
    assert "not reached" not in r.stdout and "exceeded the 0.5 s deadline" in r.stderr


def test_run_accepts_a_prefetched_feed_on_a_cpu_session():
    """``prefetch=`` is an upload hint: on a CPU session nothing is copied ahead and the results are those of plain feeding."""
    import torch
    from autodist_b200.strategy import PS
    values = []
    for use in (False, True):
        _reset_default_autodist()
        ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=PS())
        with ad.scope():
            torch.manual_seed(0)
            w = torch.nn.Parameter(torch.zeros(3))
            x = ad.placeholder((None, 3), torch.float32, name="x")
            loss = ((x * w).sum(1) - 1.0).pow(2).mean()
            train_op = torch.optim.SGD([w], lr=0.1).minimize(loss)
            sess = ad.create_distributed_session()
            batches = [torch.full((4, 3), float(i + 1)) for i in range(4)]
            out = []
            for i, b in enumerate(batches):
                nxt = {x: batches[i + 1]} if use and i + 1 < len(batches) else None
                out.append(float(sess.run([loss, train_op], {x: b}, prefetch=nxt)[0]))
            values.append((out, sess.run(w).tolist()))
            sess.close()
    _reset_default_autodist()
    assert values[0] == values[1]


def test_parameter_groups_keep_their_hyper_parameters_on_the_generic_engine():
    """AdamW with two groups (weight decay on the weights only, a different learning rate on the biases) through a session
    equals the same optimizer stepped by hand."""
    import copy
    import torch
    from autodist_b200.strategy import AllReduce

    def make_groups(net):
        weights = [p for n, p in net.named_parameters() if n.endswith("weight")]
        biases = [p for n, p in net.named_parameters() if n.endswith("bias")]
        return [{"params": weights, "weight_decay": 0.5}, {"params": biases, "weight_decay": 0.0, "lr": 0.05}]

    torch.manual_seed(1)
    base = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 1))
    g = torch.Generator().manual_seed(0)
    data = [(torch.randn(8, 6, generator=g), torch.randn(8, 1, generator=g)) for _ in range(5)]

    ref = copy.deepcopy(base)
    opt = torch.optim.AdamW(make_groups(ref), lr=0.01)
    for xb, yb in data:
        opt.zero_grad()
        ((ref(xb) - yb) ** 2).mean().backward()
        opt.step()

    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=AllReduce())
    with ad.scope():
        net = copy.deepcopy(base)
        x = ad.placeholder((None, 6), torch.float32, name="x")
        y = ad.placeholder((None, 1), torch.float32, name="y")
        loss = ((net(x) - y) ** 2).mean()
        train_op = torch.optim.AdamW(make_groups(net), lr=0.01).minimize(loss)
        sess = ad.create_distributed_session()
        for xb, yb in data:
            sess.run(train_op, {x: xb, y: yb})
        got = {n: torch.from_numpy(sess.run(p)) for n, p in net.named_parameters()}
        sess.close()
    _reset_default_autodist()
    for n, p in ref.named_parameters():
        assert torch.allclose(got[n], p.detach(), atol=1e-6), n


def test_two_train_ops_of_two_optimizers_in_one_run_call():
    """Two networks with their own optimizers fetched together: both gradients are taken at the values before the call,
    as when the same is written by hand; train ops over the same variables are refused."""
    import copy
    import torch
    from autodist_b200.strategy import AllReduce
    torch.manual_seed(2)
    enc0, head0 = torch.nn.Linear(5, 4), torch.nn.Linear(4, 1)
    g = torch.Generator().manual_seed(0)
    data = [(torch.randn(8, 5, generator=g), torch.randn(8, 1, generator=g)) for _ in range(4)]

    enc, head = copy.deepcopy(enc0), copy.deepcopy(head0)
    o1, o2 = torch.optim.SGD(enc.parameters(), lr=0.1), torch.optim.Adam(head.parameters(), lr=0.01)
    for xb, yb in data:
        h = torch.tanh(enc(xb))
        l1, l2 = (h ** 2).mean(), ((head(h) - yb) ** 2).mean()
        o1.zero_grad(); o2.zero_grad()
        l1.backward(inputs=list(enc.parameters()), retain_graph=True)
        l2.backward(inputs=list(head.parameters()))
        o1.step(); o2.step()

    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=AllReduce())
    with ad.scope():
        e, hd = copy.deepcopy(enc0), copy.deepcopy(head0)
        x = ad.placeholder((None, 5), torch.float32, name="x")
        y = ad.placeholder((None, 1), torch.float32, name="y")
        hidden = torch.tanh(e(x))
        loss1, loss2 = (hidden ** 2).mean(), ((hd(hidden) - y) ** 2).mean()
        op1 = torch.optim.SGD(e.parameters(), lr=0.1).minimize(loss1, var_list=list(e.parameters()))
        op2 = torch.optim.Adam(hd.parameters(), lr=0.01).minimize(loss2, var_list=list(hd.parameters()))
        both = torch.optim.SGD(list(e.parameters()) + list(hd.parameters()), lr=0.1).minimize(loss2)
        sess = ad.create_distributed_session()
        for xb, yb in data:
            l1v, l2v, _, _ = sess.run([loss1, loss2, op1, op2], {x: xb, y: yb})
        got = {("e", n): torch.from_numpy(sess.run(p)) for n, p in e.named_parameters()}
        got.update({("h", n): torch.from_numpy(sess.run(p)) for n, p in hd.named_parameters()})
        with pytest.raises(NotImplementedError):
            sess.run([op1, both], {x: data[0][0], y: data[0][1]})
        sess.close()
    _reset_default_autodist()
    for n, p in enc.named_parameters():
        assert torch.allclose(got[("e", n)], p.detach(), atol=1e-6), n
    for n, p in head.named_parameters():
        assert torch.allclose(got[("h", n)], p.detach(), atol=1e-6), n
