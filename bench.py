"""Headline benchmark: BERT-large pre-training throughput (sequences/s), seq 128, batch 32 per GPU.

``python bench.py --gpus N --steps K --warmup W`` (N > 1: launched by ``torch.distributed.run``, one rank
per GPU). Runs the training step through the framework's public API (``AutoDist`` -> ``scope`` ->
``create_distributed_session`` -> ``sess.run``) on synthetic data with random-initialised weights and prints
ONE JSON line on rank 0. ``value`` is device-timed with inputs resident on the device; ``e2e`` repeats the
measurement with every step's inputs copied from pinned host memory and the loss read back to the host.
``--impl reference`` reports why the reference itself cannot run here.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# per-GPU examples/s of the reference's "AutoDist AllReduce" BERT-large bars (T4, read off docs/usage/figure1.png)
PUBLISHED_PER_GPU = {1: 11.1, 2: 8.0, 4: 7.8, 8: 3.2}
PUBLISHED_RESNET101 = {1: 62.0, 2: 59.5, 4: 59.0, 8: 52.0}     # images/s/GPU, "AutoDist AllReduce" bars


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self._stop_evt = index, [], threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            for line in self.proc.stdout:
                self.samples.append([x.strip() for x in line.split(",")])
                if self._stop_evt.is_set():
                    break
        except (OSError, ValueError):
            pass

    def stop(self):
        self._stop_evt.set()
        if self.proc is not None:
            self.proc.terminate()     # the exact process this thread started

    def summary(self):
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return 0                      # one line per job, from rank 0
    print(json.dumps({
        "impl": "reference",
        "unavailable": "petuum/autodist needs TensorFlow 1.15-2.2 (CUDA 10, no sm_100 code) and protoc at install time; "
                       "neither is present offline: the offline pip install of the reference stops in its setup.py generate_proto step"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="bert-large", choices=["bert-large", "bert-base", "bert-tiny", "resnet101", "vgg16",
                                                              "resnet50", "densenet121", "inceptionv3", "lm1b", "lm1b-tiny"])
    ap.add_argument("--strategy", default="allreduce", choices=["allreduce", "allreduce_ef", "parallax", "ps", "partitioned_ps"])
    ap.add_argument("--batch", type=int, default=0, help="samples per GPU (default: 32 sequences, 64 images, 32 for vgg16)")
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--comm", default=None, help="fused (own kernels) or nccl (baseline)")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.comm:
        os.environ["AUTODIST_COMM"] = args.comm
    if args.no_graph:
        os.environ["AUTODIST_CUDA_GRAPH"] = "0"
    os.environ.setdefault("AUTODIST_MIN_LOG_LEVEL", "WARNING")
    os.environ.setdefault("AUTODIST_FETCH_MODE", "local")
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from autodist_b200 import AutoDist, ops
    from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200 import strategy as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    n_gpus = args.gpus
    if world != n_gpus and world > 1:
        n_gpus = world
    builders = {
        "allreduce": lambda: S.AllReduce(chunk_size=256),
        "allreduce_ef": lambda: S.AllReduce(chunk_size=256, compressor="HorovodCompressorEF"),
        "parallax": lambda: S.Parallax(chunk_size=256, reduction_devices="gpu"),
        "ps": lambda: S.PSLoadBalancing(reduction_devices="gpu", local_proxy_variable=True),
        "partitioned_ps": lambda: S.PartitionedPS(num_shards=n_gpus, reduction_devices="gpu", local_proxy_variable=True),
    }
    is_bert = args.model.startswith("bert")
    is_lm = args.model.startswith("lm1b")
    if not args.batch:
        args.batch = 128 if is_lm else (32 if is_bert or args.model == "vgg16" else 64)
    max_pred = 20
    ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=n_gpus), strategy_builder=builders[args.strategy]())
    # Every process feeds its node's whole batch (batch per GPU x GPUs of the node), as a user of the API does; the
    # remapper keeps this replica's slice, so only that slice crosses PCIe.
    if is_bert:
        cfg = {"bert-large": BertConfig.large, "bert-base": BertConfig.base, "bert-tiny": BertConfig.tiny}[args.model]()
        host_batches = [synthetic_batch(cfg, args.batch * n_gpus, args.seq, max_pred, seed=i, pin=True) for i in range(4)]
    elif is_lm:
        from autodist_b200.models.lm1b import LM1B, LM1BConfig, zipf_tokens
        cfg = LM1BConfig.tiny() if args.model == "lm1b-tiny" else LM1BConfig()
        host_batches = [{k: v.pin_memory() for k, v in zipf_tokens(args.batch * n_gpus, cfg.num_steps, cfg.vocab_size, seed=i).items()}
                        for i in range(4)]
    else:
        from autodist_b200.models.cnn import ImageClassifier, synthetic_images
        host_batches = [{k: v.pin_memory() for k, v in synthetic_images(args.batch * n_gpus, 224, 1000, seed=i).items()}
                        for i in range(2)]
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values()) // n_gpus
    with ad.scope():
        torch.manual_seed(0)
        model = BertPretrainer(cfg) if is_bert else LM1B(cfg) if is_lm else (ImageClassifier(args.model, image_size=224) if args.model == "vgg16"
                                                     else ImageClassifier(args.model))
        phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in host_batches[0].items()}
        loss = model(**phs)
        if is_lm:
            opt = torch.optim.Adagrad(model.parameters(), lr=0.2, initial_accumulator_value=1.0)
            train_op = opt.minimize(loss, clip_global_norm=(cfg.max_grad_norm, model.dense_parameters()))
        else:
            opt = torch.optim.Adam(model.parameters(), lr=1e-4) if is_bert else \
                torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
            train_op = opt.minimize(loss)
        sess = ad.create_distributed_session()
        dev = sess.engine.device
        dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches]

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def feed(batches, i):
            b = batches[i % len(batches)]
            return {phs[k]: b[k] for k in phs}

        # ---- warm-up (also builds workspaces and captures the CUDA graph)
        for i in range(args.warmup + 3):
            sess.run(train_op, feed(dev_batches, i))
        for i in range(2):                                   # the end-to-end form of the call is warmed up as well
            sess.run([loss, train_op], feed(host_batches, i))
        sess.engine.check_errors() if hasattr(sess.engine, "check_errors") else None

        sampler = ClockSampler(dev.index or 0) if rank == 0 else None
        if sampler:
            sampler.start()
            time.sleep(0.3)
        # ---- device-timed region: K steps, inputs resident on the device
        launches0 = ops.launch_count
        per_step_launches = getattr(sess.engine, "launches_per_step", 0)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            sess.run(train_op, feed(dev_batches, i))
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        eager_launches = ops.launch_count - launches0
        # ---- end-to-end region: pinned host inputs copied every step, loss read back every step
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        last = None
        for i in range(args.steps):
            last, _ = sess.run([loss, train_op], feed(host_batches, i))
        f1.record()
        barrier()
        ms_e2e = f0.elapsed_time(f1)
        if sampler:
            sampler.stop()
        if hasattr(sess.engine, "check_errors"):
            sess.engine.check_errors()

        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    if rank != 0:
        return 0
    global_batch = args.batch * n_gpus
    per_sample = cfg.num_steps if is_lm else 1                 # LM1B counts words: batch x unrolled steps
    value = global_batch * per_sample * args.steps / (ms / 1e3)
    e2e = global_batch * per_sample * args.steps / (ms_e2e / 1e3)
    unit = "sequences/s" if is_bert else "words/s" if is_lm else "images/s"
    graph_launches = getattr(sess.engine, "graph_kernels", 0)
    launches = eager_launches if eager_launches > 0 else graph_launches * args.steps
    published = PUBLISHED_PER_GPU.get(n_gpus)
    out = {
        "metric": "BERT-large pre-training sequences/sec (seq 128), max over ranks" if is_bert
        else "LM1B big-LSTM training words/sec (20 unrolled steps, sampled softmax 8192), max over ranks" if is_lm
        else f"{args.model} ImageNet-shape training images/sec, max over ranks",
        "value": round(value, 2), "unit": unit, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / (published * n_gpus), 2) if published and args.model == "bert-large" else (
            round(value / (PUBLISHED_RESNET101.get(n_gpus, 0) * n_gpus), 2) if args.model == "resnet101" and n_gpus in PUBLISHED_RESNET101 else None),
        "dtype": "bf16", "data": "synthetic (uniform token ids, 15% MLM positions, random-init weights)" if is_bert
        else "synthetic (Zipf(1.1) token ids over the 793471-word vocabulary, random-init weights)" if is_lm else "synthetic (images ~ N(0,1), uniform labels over 1000 classes, random-init weights)",
        "config": {"model": args.model, "global_batch": global_batch, "seq_len": args.seq if is_bert else (cfg.num_steps if is_lm else None),
                   "max_predictions": max_pred if is_bert else None,
                   "compute": "hand-written sm_100a kernels" if is_bert else "tcgen05 GEMM + own LSTM-cell / gather kernels, autograd glue" if is_lm else "tcgen05 implicit-GEMM convolutions (forward, dgrad, wgrad) + own batch-norm / ReLU / max-pool kernels + tcgen05 GEMM for fully connected layers" if os.environ.get("AUTODIST_CONV", "own") != "library" else "library convolutions + own batch-norm / ReLU / max-pool kernels + tcgen05 GEMM for fully connected layers",
                   "parallelism": f"dp{n_gpus}", "strategy": args.strategy, "optimizer": "Adam, fp32 master + bf16 compute" if is_bert else "Adagrad 0.2, LSTM gradients clipped at norm 10" if is_lm else "SGD momentum 0.9, fp32 master + bf16 autocast",
                   "comm": os.environ.get("AUTODIST_COMM", "fused"),
                   "cuda_graph": os.environ.get("AUTODIST_CUDA_GRAPH", "1") != "0",
                   "l2": "per-step working set (activations + weights > 4 GB) is far larger than the 126 MB L2",
                   "engine": type(sess.engine).__name__},
        "clocks": sampler.summary() if sampler else None,
        "e2e": {"value": round(e2e, 2), "unit": unit, "ms_per_step": round(ms_e2e / args.steps, 3),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": float(last)},
        "gpu_launches": int(launches),
        "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
