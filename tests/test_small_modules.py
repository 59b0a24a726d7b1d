"""Units with only indirect coverage elsewhere: flat parameter storage, optimizer tables, stage dumps."""
import os

import pytest
import torch
from torch import nn


def test_flat_params_layout_and_views():
    from autodist_b200.ops.flat import FlatParams
    torch.manual_seed(0)
    mods = nn.ModuleDict({"a": nn.Linear(3, 5), "b": nn.Linear(5, 1)})            # numels 15, 5, 5, 1: none a multiple of 8
    named = list(mods.named_parameters())
    before = {n: p.detach().clone() for n, p in named}
    fl = FlatParams(named, "cpu")
    assert fl.total % 64 == 0
    for n, p in named:
        assert fl.offsets[n] % 8 == 0                                            # 16-byte boundary in bf16, 32 in fp32
        assert p.data.data_ptr() == fl.w32[n].data_ptr() and p.grad.data_ptr() == fl.g[n].data_ptr()
        torch.testing.assert_close(fl.w32[n], before[n])
        torch.testing.assert_close(fl.w16[n].float(), before[n], rtol=1e-2, atol=1e-2)
    lo, hi = fl.range_of(["a.weight", "a.bias"])
    assert lo == 0 and hi == fl.offsets["b.weight"]
    assert fl.range_of(["b.bias"])[1] == fl.total
    # autograd accumulates straight into the flat gradient buffer
    fl.grad.zero_()
    x = torch.randn(4, 3)
    mods["b"](mods["a"](x)).sum().backward()
    assert fl.grad.abs().sum() > 0 and mods["a"].weight.grad.data_ptr() == fl.g["a.weight"].data_ptr()
    new_grad = torch.zeros(fl.total)
    fl.rebind_grad(new_grad)
    assert mods["a"].weight.grad.data_ptr() == new_grad.data_ptr()
    fl.master[:15].add_(1.0)
    fl.refresh_bf16()
    torch.testing.assert_close(fl.w16["a.weight"].float(), fl.w32["a.weight"], rtol=1e-2, atol=1e-2)


def test_optimizer_tables():
    from autodist_b200.kernel.common import op_info
    assert op_info.slot_names(torch.optim.Adam) == ("exp_avg", "exp_avg_sq") or "exp_avg" in op_info.slot_names(torch.optim.Adam)
    p = [nn.Parameter(torch.zeros(2))]
    assert op_info.supports_sparse_rows(torch.optim.SGD(p, lr=0.1))
    assert not op_info.supports_sparse_rows(torch.optim.SGD(p, lr=0.1, momentum=0.9))
    assert not op_info.supports_sparse_rows(torch.optim.SGD(p, lr=0.1, weight_decay=0.1))
    assert op_info.supports_sparse_rows(torch.optim.Adagrad(p, lr=0.1))
    assert not op_info.supports_sparse_rows(torch.optim.Adam(p, lr=0.1))
    assert set(op_info.FUSED) <= set(op_info.DENSE_UPDATE_OPTIMIZERS)


def test_stage_dumps_and_dot_export(tmp_path, monkeypatch):
    import torch.fx
    from autodist_b200 import const
    from autodist_b200.utils import visualization_util as vz
    monkeypatch.setattr(const, "DEFAULT_GRAPH_DIR", str(tmp_path / "graphs"))
    monkeypatch.delenv("AUTODIST_DUMP_GRAPHS", raising=False)
    assert vz.log_graph("x", "0-original") is None

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Parameter(torch.ones(2))

        def forward(self, x):
            return (x * self.w).sum()

    gm = torch.fx.symbolic_trace(M())
    dot = vz.fx_graph_to_dot(gm.graph, "m")
    assert dot.startswith('digraph "m" {') and dot.rstrip().endswith("}")
    assert '"x" -> "mul"' in dot and "shape=box" in dot and "shape=octagon" in dot and "shape=doublecircle" in dot
    monkeypatch.setenv("AUTODIST_DUMP_GRAPHS", "1")
    p1 = vz.log_graph("plan text", "3-transformed")
    p2 = vz.log_fx_graph(gm.graph, "0-original")
    assert open(p1).read() == "plan text" and p1.endswith(f"3-transformed.{os.getpid()}.txt")
    assert open(p2).read() == vz.fx_graph_to_dot(gm.graph, "0-original")


def test_transformer_writes_all_four_stages(tmp_path, monkeypatch):
    from autodist_b200 import AutoDist, const
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import PartitionedPS
    monkeypatch.setattr(const, "DEFAULT_GRAPH_DIR", str(tmp_path / "graphs"))
    monkeypatch.setenv("AUTODIST_DUMP_GRAPHS", "1")
    monkeypatch.setenv("AUTODIST_IS_TESTING", "True")
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=PartitionedPS())
    with ad.scope():
        w = nn.Parameter(torch.zeros(6, 2))
        x = ad.placeholder((None, 6), torch.float32, name="x")
        loss = (x @ w).pow(2).mean()
        torch.optim.SGD([w], lr=0.1).minimize(loss)
        sess = ad.create_distributed_session()
        sess.close()
    _reset_default_autodist()
    names = sorted(os.listdir(tmp_path / "graphs"))
    stages = {n.split(".")[0] for n in names}
    assert stages == {"0-original", "1-after-partition", "2-after-in-graph", "3-transformed"}
    assert any(n.endswith(".dot") for n in names)


def test_bench_reference_arm_prints_one_json_line():
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE")}
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and ("unavailable" in rec or "value" in rec)
    # a non-zero rank of a multi-process launch stays silent
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"], capture_output=True, text=True,
                       timeout=300, env=dict(env, RANK="1", WORLD_SIZE="2"))
    assert r.returncode == 0 and r.stdout.strip() == ""
