"""The meeting point of the two consumers of a forked tensor (``ops/functional.py``: ``GradFork`` / ``_ForkFn``), exercised
on CPU with stand-in consumers: on a GPU the consumers are the input-gradient convolution and the batch-norm backward."""
import torch

from autodist_b200.ops.functional import GradFork, _ForkFn, fork


class _Consumer(torch.autograd.Function):
    """``y = scale * x``. With a ``GradFork``: the first backward to run leaves its gradient there and returns none, the
    second adds what it finds (the stand-in for an epilogue add) and returns the sum."""

    @staticmethod
    def forward(ctx, x, scale, box, log):
        ctx.scale, ctx.box, ctx.log = scale, box, log
        return x * scale

    @staticmethod
    def backward(ctx, g):
        mine = g * ctx.scale
        if ctx.box is None:
            return mine, None, None, None
        other = ctx.box.take()
        if other is None:
            ctx.log.append(("left", ctx.scale))
            ctx.box.grad = mine
            return None, None, None, None
        ctx.log.append(("added", ctx.scale))
        return mine + other, None, None, None


def test_fork_on_cpu_is_the_identity():
    x = torch.randn(3, requires_grad=True)
    a, b, box = fork(x)
    assert a is x and b is x and box is None


def test_second_consumer_adds_the_first_ones_gradient():
    x = torch.randn(5, requires_grad=True)
    box, log = GradFork(), []
    xin = x * 1.0
    a, b = _ForkFn.apply(xin, box)
    y = _Consumer.apply(a, 2.0, box, log) + _Consumer.apply(b, 3.0, box, log)
    g = torch.randn(5)
    y.backward(g)
    assert torch.allclose(x.grad, 5.0 * g)
    assert [kind for kind, _ in log] == ["left", "added"] and box.grad is None


def test_a_consumer_that_does_not_know_the_fork_still_gets_its_gradient_counted():
    x = torch.randn(5, requires_grad=True)
    box, log = GradFork(), []
    a, b = _ForkFn.apply(x * 1.0, box)
    y = _Consumer.apply(a, 2.0, box, log) + b * 7.0             # the second consumer is ordinary autograd
    g = torch.randn(5)
    y.backward(g)
    assert torch.allclose(x.grad, 9.0 * g)                      # the gradient left in the fork is picked up by the fork itself
    assert log == [("left", 2.0)] and box.grad is None


def test_a_branch_without_gradient_does_not_lose_the_other():
    x = torch.randn(5, requires_grad=True)
    box, log = GradFork(), []
    a, b = _ForkFn.apply(x * 1.0, box)
    y = _Consumer.apply(a, 2.0, box, log) + _Consumer.apply(b, 3.0, box, log).detach()
    g = torch.randn(5)
    y.backward(g)
    assert torch.allclose(x.grad, 2.0 * g)
