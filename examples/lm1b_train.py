"""LM1B language-model training on synthetic Zipf token ids (reference: ``examples/lm1b/lm1b_train.py``).

Uses the decorator-style entry point: ``ad.function(train_step)`` traces once, then every call is one distributed step.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist, strategy as S  # noqa: E402
from autodist_b200.models.lm1b import LM1B, LM1BConfig, zipf_tokens  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--batch_size", type=int, default=128, help="per GPU")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--strategy", default="PartitionedPS", choices=["PS", "PartitionedPS", "AllReduce", "Parallax"])
    args = ap.parse_args()
    n = args.gpus
    cfg = LM1BConfig.tiny() if args.tiny else LM1BConfig()
    builder = {"PS": lambda: S.PS(), "PartitionedPS": lambda: S.PartitionedPS(num_shards=max(n, 2), reduction_devices="gpu"),
               "AllReduce": lambda: S.AllReduce(), "Parallax": lambda: S.Parallax()}[args.strategy]()
    spec = ResourceSpec.local(num_gpus=n if torch.cuda.is_available() else 0, num_cpus=n)
    ad = AutoDist(resource_spec=spec, strategy_builder=builder)
    data = zipf_tokens(args.batch_size * n, cfg.num_steps, cfg.vocab_size)
    with ad.scope():
        model = LM1B(cfg)
        opt = torch.optim.Adagrad(model.parameters(), lr=0.2, initial_accumulator_value=1.0)

        @ad.function
        def train_step(x, y):
            loss = model(x, y)
            return loss, opt.minimize(loss, clip_global_norm=(cfg.max_grad_norm, model.dense_parameters()))

        t0 = time.time()
        for step in range(1, args.steps + 1):
            loss, _ = train_step(data["x"], data["y"])
            if ad.rank == 0 and step % 10 == 0:
                wps = 10 * args.batch_size * n * cfg.num_steps / (time.time() - t0)
                print(f"step {step} loss {float(loss):.3f} {wps:.0f} words/s", flush=True)
                t0 = time.time()


if __name__ == "__main__":
    main()
