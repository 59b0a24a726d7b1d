"""Several optimizer parameter groups (their own learning rate / weight decay) on the fused engines: the flat-buffer update
must apply each group's hyper-parameters to exactly that group's parameters."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(opt_name, fused):
    import os
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import AllReduce
    os.environ["AUTODIST_COMM"] = "fused" if fused else "nccl"
    try:
        _reset_default_autodist()
        ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=1), strategy_builder=AllReduce(chunk_size=2))
        with ad.scope():
            torch.manual_seed(3)
            net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 16), torch.nn.Tanh(), torch.nn.Linear(16, 1))
            x = ad.placeholder((None, 32), torch.float32, name="x")
            y = ad.placeholder((None, 1), torch.float32, name="y")
            loss = ((net(x) - y) ** 2).mean()
            weights = [p for n, p in net.named_parameters() if n.endswith("weight")]
            biases = [p for n, p in net.named_parameters() if n.endswith("bias")]
            groups = [{"params": weights, "weight_decay": 5.0}, {"params": biases, "weight_decay": 0.0, "lr": 0.05}]
            if opt_name == "adamw":
                opt = torch.optim.AdamW(groups, lr=0.01)
            else:
                opt = torch.optim.SGD(groups, lr=0.02, momentum=0.9)
            train_op = opt.minimize(loss)
            sess = ad.create_distributed_session()
            engine = type(sess.engine).__name__
            g = torch.Generator().manual_seed(0)
            for step in range(6):
                xb, yb = torch.randn(16, 32, generator=g), torch.randn(16, 1, generator=g)
                if step == 3:
                    opt.param_groups[1]["lr"] = 0.005                 # a schedule that moves one group only
                sess.run(train_op, {x: xb, y: yb})
            values = {n: torch.from_numpy(sess.run(p)).clone() for n, p in net.named_parameters()}
            sess.close()
        return engine, values
    finally:
        os.environ.pop("AUTODIST_COMM", None)
        _reset_default_autodist()


@pytest.mark.parametrize("opt_name", ["adamw", "sgd"])
def test_parameter_groups_on_the_fused_engine_match_the_torch_optimizer(opt_name):
    fused_engine, fused = _run(opt_name, True)
    generic_engine, generic = _run(opt_name, False)
    assert fused_engine == "FlatAutogradEngine" and generic_engine == "StepEngine", (fused_engine, generic_engine)
    for n in fused:
        # a group that got the other group's weight decay (5 against 0) or learning rate (0.05 against 0.01 / 0.02) is off by
        # tens of percent after six steps; rounding differences between the two optimizer implementations are far below 1 %
        diff = (fused[n] - generic[n]).abs().max().item()
        scale = generic[n].abs().max().item() + 1e-3
        assert diff <= 0.01 * scale + 1e-4, (n, diff, scale)
