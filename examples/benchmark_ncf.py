"""NeuMF (NCF) training on synthetic ml-20m-shaped interactions (reference: ``examples/benchmark/ncf.py``)."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist  # noqa: E402
from autodist_b200.models.ncf import NeuMF, NeuMFConfig, hit_rate_and_ndcg, synthetic_interactions  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402
from autodist_b200.utils import train_utils as tu  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    tu.add_base_flags(ap, batch_size=16384, train_steps=60)
    tu.add_benchmark_flags(ap, log_steps=20)
    tu.add_strategy_flags(ap, default="Parallax")
    ap.add_argument("--optimizer", default="adam", choices=["adam", "sgd", "lazy_adam"])
    ap.add_argument("--learning_rate", type=float, default=0.001)
    ap.add_argument("--dense_gradient", action="store_true", help="dense embedding gradients (for all-reduce strategies)")
    ap.add_argument("--tiny", action="store_true")
    args = ap.parse_args()
    n = args.gpus
    cfg = NeuMFConfig.tiny(dense_gradient=args.dense_gradient) if args.tiny else NeuMFConfig(dense_gradient=args.dense_gradient)
    spec = ResourceSpec(args.resource_spec) if args.resource_spec else \
        ResourceSpec.local(num_gpus=n if torch.cuda.is_available() else 0, num_cpus=n)
    ad = AutoDist(resource_spec=spec, strategy_builder=tu.build_strategy(args.autodist_strategy, args.chunk_size, args.compressor, n))
    data = synthetic_interactions(args.batch_size * n, cfg)
    logger = tu.MetricsLogger(args.benchmark_log, stream=None)
    logger.log_run_info("neumf", "synthetic ml-20m shape", vars(args))
    with ad.scope():
        model = NeuMF(cfg)
        phs = {k: ad.placeholder((None,), v.dtype, name=k) for k, v in data.items()}
        loss = model(**phs)
        if args.optimizer == "sgd":
            opt = torch.optim.SGD(model.parameters(), lr=args.learning_rate)
        elif args.optimizer == "lazy_adam" and not args.dense_gradient:
            opt = torch.optim.SparseAdam(model.sparse_grad_parameters(), lr=args.learning_rate)
            opt2 = torch.optim.Adam([p for p in model.parameters() if all(p is not q for q in model.sparse_grad_parameters())],
                                    lr=args.learning_rate)
        else:
            opt = torch.optim.Adam(model.parameters(), lr=args.learning_rate)
        train_ops = [opt.minimize(loss)]
        if args.optimizer == "lazy_adam" and not args.dense_gradient:
            train_ops.append(opt2.minimize(loss))
        sess = ad.create_distributed_session()
        hist = tu.TimeHistory(args.batch_size * n, args.log_steps)
        hist.on_train_begin()
        for _ in range(args.train_steps):
            lv = sess.run([loss] + train_ops, {phs[k]: data[k] for k in phs})[0]
            rec = hist.on_step_end()
            if rec and sess.rank == 0:
                print(f"step {rec['step']} loss {float(lv):.4f} {rec['examples_per_sec']:.0f} examples/s", flush=True)
                logger.log_metric("examples_per_sec", rec["examples_per_sec"], "examples/s", rec["step"])
        if sess.rank == 0:
            # leave-one-out style evaluation on synthetic candidates: 1 positive column + 99 sampled negatives
            with torch.no_grad():
                dev = next(model.parameters()).device
                users = torch.randint(0, cfg.num_users, (256,), device=dev)
                items = torch.randint(0, cfg.num_items, (256, 100), device=dev)
                scores = model.logits(users[:, None].expand(-1, 100).reshape(-1), items.reshape(-1)).view(256, 100)
                hr, ndcg = hit_rate_and_ndcg(scores.float().cpu())
                print(f"HR@10 {hr:.3f} NDCG@10 {ndcg:.3f} (synthetic candidates)", flush=True)


if __name__ == "__main__":
    main()
