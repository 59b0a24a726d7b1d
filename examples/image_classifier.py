"""Getting-started CNN on Fashion-MNIST-shaped synthetic data with the default strategy
(reference: ``examples/image_classifier.py``)."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist  # noqa: E402
from autodist_b200.models.simple import FashionCNN  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402


def fit_route(ad, images, labels):
    """The same model through ``compile / fit / evaluate`` (the counterpart of the reference's Keras route)."""
    from autodist_b200.training import Model
    model = Model(ad, FashionCNN)
    model.compile(optimizer=lambda params: torch.optim.SGD(params, lr=0.05), loss=torch.nn.functional.cross_entropy,
                  metrics={"accuracy": lambda out, y: (out.argmax(1) == y).float().mean()})
    model.fit(images, labels, batch_size=64, epochs=3, verbose=1)
    result = model.evaluate(images, labels, batch_size=64)   # every rank takes part: fetches are gathered across replicas
    if model.session.rank == 0:
        print("evaluate:", result)


def feeder_route(ad, images, labels):
    """The same training from a record file: native worker threads assemble the shuffled batches in pinned buffers, and
    every ``run`` starts the upload of the batch after the one it trains on."""
    import tempfile
    from autodist_b200.utils.data import RecordFeeder, write_records
    path = os.path.join(tempfile.mkdtemp(), "fashion.rec")
    write_records(path, {"images": images, "labels": labels})
    with ad.scope():
        model = FashionCNN()
        x = ad.placeholder((None, 1, 28, 28), torch.float32, name="images")
        y = ad.placeholder((None,), torch.int64, name="labels")
        loss = model(x, y)
        train_op = torch.optim.SGD(model.parameters(), lr=0.05).minimize(loss)
        sess = ad.create_distributed_session()
        # every process feeds its node's batches; the session splits them between the node's replicas
        batches = iter(RecordFeeder(path, 64, shuffle=True, seed=0, epochs=5, depth=3))
        current, step = next(batches), 0
        while current is not None:
            upcoming = next(batches, None)
            lv, _ = sess.run([loss, train_op], {x: current["images"], y: current["labels"]},
                             prefetch=None if upcoming is None else {x: upcoming["images"], y: upcoming["labels"]})
            if sess.rank == 0 and step % 4 == 0:
                print(f"step {step} loss {float(lv):.4f}")
            current, step = upcoming, step + 1


def main():
    args = [a for a in sys.argv[1:] if a not in ("--fit", "--feeder")]
    spec = ResourceSpec(args[0]) if args else ResourceSpec.local(num_cpus=2)
    ad = AutoDist(resource_spec=spec)                     # default builder: PSLoadBalancing
    rng = np.random.RandomState(0)
    images = rng.rand(256, 1, 28, 28).astype(np.float32)
    labels = rng.randint(0, 10, size=256).astype(np.int64)
    if "--fit" in sys.argv:
        return fit_route(ad, images, labels)
    if "--feeder" in sys.argv:
        return feeder_route(ad, images, labels)
    with ad.scope():
        model = FashionCNN()
        x = ad.placeholder((None, 1, 28, 28), torch.float32, name="images")
        y = ad.placeholder((None,), torch.int64, name="labels")
        loss = model(x, y)
        train_op = torch.optim.SGD(model.parameters(), lr=0.05).minimize(loss)
        sess = ad.create_distributed_session()
        for epoch in range(5):
            lv, _ = sess.run([loss, train_op], {x: images, y: labels})
            if sess.rank == 0:
                print(f"epoch {epoch} loss {float(lv):.4f}")


if __name__ == "__main__":
    main()
