"""ImageNet-shape CNN benchmark on synthetic data (reference: ``examples/benchmark/imagenet.py``).

``python examples/benchmark_imagenet.py --cnn_model resnet101 --autodist_strategy AllReduce --gpus 8``
(or under ``torchrun``). Prints images/s every ``--log_steps`` steps.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from autodist_b200 import AutoDist, strategy as S  # noqa: E402
from autodist_b200.models.cnn import ImageClassifier, synthetic_images  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402
from autodist_b200.utils import train_utils as tu  # noqa: E402

# variables per collective group used by the reference's driver (imagenet.py:151-158)
CHUNK = {"vgg16": 25, "resnet101": 200, "inceptionv3": 30}


def build_strategy(name, chunk, n):
    return {
        "PS": lambda: S.PS(), "PSLoadBalancing": lambda: S.PSLoadBalancing(),
        "PartitionedPS": lambda: S.PartitionedPS(num_shards=n, reduction_devices="gpu"),
        "UnevenPartitionedPS": lambda: S.UnevenPartitionedPS(reduction_devices="gpu"),
        "AllReduce": lambda: S.AllReduce(chunk_size=chunk),
        "AllReduceEF": lambda: S.AllReduce(chunk_size=chunk, compressor="HorovodCompressorEF"),
        "PowerSGD": lambda: S.AllReduce(chunk_size=chunk, compressor="PowerSGDCompressor", power_sgd_rank=1),
        "PartitionedAR": lambda: S.PartitionedAR(chunk_size=chunk),
        "RandomAxisPartitionAR": lambda: S.RandomAxisPartitionAR(chunk_size=chunk),
        "Parallax": lambda: S.Parallax(chunk_size=chunk),
    }[name]()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cnn_model", default="resnet101", choices=["resnet101", "resnet50", "vgg16", "inceptionv3", "densenet121"])
    ap.add_argument("--autodist_strategy", default="AllReduce")
    ap.add_argument("--resource_spec", default="")
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--batch_size", type=int, default=64, help="per GPU")
    ap.add_argument("--image_size", type=int, default=224)
    ap.add_argument("--train_steps", type=int, default=50)
    ap.add_argument("--log_steps", type=int, default=10)
    ap.add_argument("--chunk_size", type=int, default=0)
    ap.add_argument("--lr_schedule", action="store_true",
                    help="warm-up + piecewise-constant decay (30/60/80 epochs) instead of a fixed rate")
    ap.add_argument("--benchmark_log", default=None, help="JSONL metrics file")
    args = ap.parse_args()
    spec = ResourceSpec(args.resource_spec) if args.resource_spec else ResourceSpec.local(
        num_gpus=args.gpus if torch.cuda.is_available() else 0, num_cpus=args.gpus)
    chunk = args.chunk_size or CHUNK.get(args.cnn_model, 512)
    ad = AutoDist(resource_spec=spec, strategy_builder=build_strategy(args.autodist_strategy, chunk, args.gpus))
    local = args.batch_size * max(1, len(spec.replica_devices))     # fed per node, split between its replicas
    data = synthetic_images(local, args.image_size)
    with ad.scope():
        model = ImageClassifier(args.cnn_model, image_size=args.image_size) if args.cnn_model == "vgg16" \
            else ImageClassifier(args.cnn_model)
        images = ad.placeholder((None, 3, args.image_size, args.image_size), torch.float32, name="images")
        labels = ad.placeholder((None,), torch.int64, name="labels")
        loss = model(images, labels)
        opt = torch.optim.SGD(model.parameters(), lr=0.01 if args.cnn_model == "vgg16" else 0.1, momentum=0.9)
        train_op = opt.minimize(loss)
        sess = ad.create_distributed_session()
        global_batch = args.batch_size * args.gpus
        sched = tu.PiecewiseConstantDecayWithWarmup(global_batch, 1281167, 5, [30, 60, 80], [1.0, 0.1, 0.01, 0.001],
                                                    base_lr=0.01 if args.cnn_model == "vgg16" else 0.1) if args.lr_schedule else None
        hist = tu.TimeHistory(global_batch, args.log_steps)
        logger = tu.MetricsLogger(args.benchmark_log) if args.benchmark_log and sess.rank == 0 else None
        if logger:
            logger.log_run_info(args.cnn_model, "synthetic ImageNet shape", vars(args))
        hist.on_train_begin()
        for step in range(1, args.train_steps + 1):
            if sched is not None:
                tu.set_learning_rate(opt, sched(step - 1))          # the engines read the captured optimizer's rate every step
            lv, _ = sess.run([loss, train_op], {images: data["images"], labels: data["labels"]})
            rec = hist.on_step_end()
            if rec and sess.rank == 0:
                print(f"step {step} loss {float(lv):.4f} {rec['examples_per_sec']:.1f} images/s", flush=True)
                if logger:
                    logger.log_metric("examples_per_sec", rec["examples_per_sec"], "images/s", step, {"loss": float(lv)})


if __name__ == "__main__":
    main()
