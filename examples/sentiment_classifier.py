"""Sentiment classifier with a partitioned, row-sparse embedding (reference: ``examples/sentiment_classifier.py``)."""
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist  # noqa: E402
from autodist_b200.models.simple import SentimentClassifier  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402
from autodist_b200.strategy import PartitionedPS  # noqa: E402


def main():
    spec = ResourceSpec(sys.argv[1]) if len(sys.argv) > 1 else ResourceSpec.local(num_cpus=2)
    ad = AutoDist(resource_spec=spec, strategy_builder=PartitionedPS())
    rng = np.random.RandomState(0)
    ids = rng.randint(0, 10000, size=(512, 256)).astype(np.int64)
    labels = (ids[:, :8].sum(1) % 2).astype(np.float32)
    with ad.scope():
        model = SentimentClassifier()
        x = ad.placeholder((None, 256), torch.int64, name="ids")
        y = ad.placeholder((None,), torch.float32, name="labels")
        loss = model(x, y)
        train_op = torch.optim.Adagrad(model.parameters(), lr=0.2).minimize(loss)
        sess = ad.create_distributed_session()
        t0 = time.time()
        for step in range(20):
            lv, _ = sess.run([loss, train_op], {x: ids, y: labels})
        if sess.rank == 0:
            print(f"loss {float(lv):.4f}  {20 * ids.size / (time.time() - t0):.0f} words/s")
            print("emb", sess.run(model.emb.weight)[:2, :4])


if __name__ == "__main__":
    main()
