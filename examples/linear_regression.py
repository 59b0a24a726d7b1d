"""Linear regression: the smallest end-to-end program (reference: ``examples/linear_regression.py``).

Run as ``python examples/linear_regression.py [resource_spec.yml]``; without an
argument a two-slot CPU spec is used (two processes over gloo).
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402
from autodist_b200.strategy import AllReduce  # noqa: E402


def make_data(n=1000, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(n).astype(np.float32)
    y = (3.0 * x + 2.0 + rng.randn(n).astype(np.float32) * 0.1).astype(np.float32)
    return x, y


def main():
    spec = ResourceSpec(sys.argv[1]) if len(sys.argv) > 1 else ResourceSpec.local(num_cpus=2)
    ad = AutoDist(resource_spec=spec, strategy_builder=AllReduce(chunk_size=128))
    x_np, y_np = make_data()
    with ad.scope():
        W = ad.variable(0.0, name="W")
        b = ad.variable(0.0, name="b")
        x = ad.placeholder((None,), torch.float32, name="x")
        y = ad.placeholder((None,), torch.float32, name="y")
        loss = ((W * x + b - y) ** 2).mean()
        opt = torch.optim.SGD([W, b], lr=0.01)
        train_op = opt.minimize(loss)
        sess = ad.create_distributed_session()
        for epoch in range(10):
            l, _ = sess.run([loss, train_op], feed_dict={x: x_np, y: y_np})
        w_val, b_val = sess.run([W, b])
        if sess.rank == 0:
            print(f"loss {float(l):.5f}  W {float(w_val):.5f}  b {float(b_val):.5f}")


if __name__ == "__main__":
    main()
