"""BERT-large pre-training benchmark on synthetic data (reference: ``examples/benchmark/bert.py``)."""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist, strategy as S  # noqa: E402
from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--autodist_strategy", default="AllReduce", choices=["AllReduce", "Parallax", "PS", "PSLoadBalancing", "PartitionedPS"])
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--train_batch_size", type=int, default=32, help="per GPU")
    ap.add_argument("--max_seq_length", type=int, default=128)
    ap.add_argument("--max_predictions_per_seq", type=int, default=20)
    ap.add_argument("--chunk_size", type=int, default=256)
    ap.add_argument("--num_train_steps", type=int, default=30)
    ap.add_argument("--learning_rate", type=float, default=5e-5)
    ap.add_argument("--model", default="large", choices=["large", "base", "tiny"])
    args = ap.parse_args()
    n = args.gpus
    builder = {"AllReduce": lambda: S.AllReduce(chunk_size=args.chunk_size), "Parallax": lambda: S.Parallax(chunk_size=args.chunk_size),
               "PS": lambda: S.PS(), "PSLoadBalancing": lambda: S.PSLoadBalancing(),
               "PartitionedPS": lambda: S.PartitionedPS(num_shards=n, reduction_devices="gpu")}[args.autodist_strategy]()
    cfg = getattr(BertConfig, args.model)()
    spec = ResourceSpec.local(num_gpus=n if torch.cuda.is_available() else 0, num_cpus=n)
    ad = AutoDist(resource_spec=spec, strategy_builder=builder)
    batch = synthetic_batch(cfg, args.train_batch_size * n, args.max_seq_length, args.max_predictions_per_seq)
    with ad.scope():
        model = BertPretrainer(cfg)
        phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in batch.items()}
        loss = model(**phs)
        opt = torch.optim.Adam(model.parameters(), lr=args.learning_rate)
        train_op = opt.minimize(loss)
        sess = ad.create_distributed_session()
        t0 = time.time()
        for step in range(1, args.num_train_steps + 1):
            lv, _ = sess.run([loss, train_op], {phs[k]: batch[k] for k in phs})
            if sess.rank == 0 and step % 10 == 0:
                print(f"step {step} loss {float(lv):.4f} {10 * args.train_batch_size * n / (time.time() - t0):.1f} examples/s", flush=True)
                t0 = time.time()


if __name__ == "__main__":
    main()
