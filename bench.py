"""Headline benchmark: BERT-large pre-training throughput (sequences/s, seq 128, batch 32 per GPU) and ResNet-101
training throughput (images/s, batch 64 per GPU).

``python bench.py --gpus N --steps K --warmup W`` (N > 1: launched by ``torch.distributed.run``, one rank
per GPU). Runs the training step through the framework's public API (``AutoDist`` -> ``scope`` ->
``create_distributed_session`` -> ``sess.run``) on synthetic data with random-initialised weights and prints
ONE JSON line on rank 0. ``value`` is device-timed with inputs resident on the device; ``e2e`` repeats the
measurement with every step's inputs copied from pinned host memory and the loss read back to the host.
The default run measures BERT-large (the line's ``value``) and, in the same call, ResNet-101 (block ``resnet101``) and
the stock-PyTorch library build of both (block ``library``: cuBLAS / cuDNN / fused SDPA / DDP, ``baseline/library_models.py``).
``--impl library`` prints the library build's own line; ``--impl reference`` reports why the reference itself cannot
run here.
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
    _emit({
        "impl": "reference",
        "unavailable": "petuum/autodist needs TensorFlow 1.15-2.2 (CUDA 10, no sm_100 code) and protoc at install time; "
                       "neither is present offline: the offline pip install of the reference stops in its setup.py generate_proto step"})
    return 0


METRIC = {"bert": "BERT-large pre-training sequences/sec (seq 128), max over ranks",
          "lm": "LM1B big-LSTM training words/sec (20 unrolled steps, sampled softmax 8192), max over ranks"}
DATA = {"bert": "synthetic (uniform token ids, 15% MLM positions, random-init weights)",
        "lm": "synthetic (Zipf(1.1) token ids over the 793471-word vocabulary, random-init weights)",
        "cnn": "synthetic (images ~ N(0,1), uniform labels over 1000 classes, random-init weights)"}
MAX_PRED = 20


def _kind(model):
    return "bert" if model.startswith("bert") else "lm" if model.startswith("lm1b") else "cnn"


def _default_batch(model):
    return 128 if model.startswith("lm1b") else (32 if model.startswith("bert") or model == "vgg16" else 64)


def _host_batches(model, batch, n_gpus, seq):
    """Pinned host batches of one node (batch per GPU x GPUs) and the configuration record of the model."""
    kind = _kind(model)
    if kind == "bert":
        from autodist_b200.models.bert import BertConfig, synthetic_batch
        cfg = {"bert-large": BertConfig.large, "bert-base": BertConfig.base, "bert-tiny": BertConfig.tiny}[model]()
        return cfg, [synthetic_batch(cfg, batch * n_gpus, seq, MAX_PRED, seed=i, pin=True) for i in range(4)]
    if kind == "lm":
        from autodist_b200.models.lm1b import LM1BConfig, zipf_tokens
        cfg = LM1BConfig.tiny() if model == "lm1b-tiny" else LM1BConfig()
        return cfg, [{k: v.pin_memory() for k, v in zipf_tokens(batch * n_gpus, cfg.num_steps, cfg.vocab_size, seed=i).items()}
                     for i in range(4)]
    from autodist_b200.models.cnn import synthetic_images
    return None, [{k: v.pin_memory() for k, v in synthetic_images(batch * n_gpus, 224, 1000, seed=i).items()} for i in range(2)]


def _timed(step_dev, step_host, steps, warmup, world, dev, sampler_rank0=True):
    """Warm-up, then K device-timed steps (inputs resident) and K end-to-end steps (pinned host inputs, loss read back), each
    bracketed by barrier + synchronize; CUDA events on the launching stream; max over ranks."""
    import torch
    import torch.distributed as dist

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup + 3):
        step_dev(i)
    for i in range(2):
        step_host(i)
    sampler = ClockSampler(dev.index or 0) if sampler_rank0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_dev(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = None
    for i in range(steps):
        last = step_host(i)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    if sampler:
        sampler.stop()
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1]), float(last), (sampler.summary() if sampler else None)


def run_ours(model_name, args, n_gpus, world, rank):
    """One measurement of the framework's own path. Returns the result record (every rank computes it)."""
    import torch
    from autodist_b200 import AutoDist, ops
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200 import strategy as S

    kind = _kind(model_name)
    batch = args.batch or _default_batch(model_name)
    strategy = args.strategy or ("parallax" if kind in ("bert", "lm") and n_gpus > 1 else "allreduce")
    builders = {
        "allreduce": lambda: S.AllReduce(chunk_size=256 if kind == "bert" else 512),
        "allreduce_ef": lambda: S.AllReduce(chunk_size=256 if kind == "bert" else 512, compressor="HorovodCompressorEF"),
        "powersgd": lambda: S.AllReduce(chunk_size=512, compressor="PowerSGDCompressor"),
        "parallax": lambda: S.Parallax(chunk_size=256, reduction_devices="gpu"),
        "ps": lambda: S.PSLoadBalancing(reduction_devices="gpu", local_proxy_variable=True),
        "partitioned_ps": lambda: S.PartitionedPS(num_shards=n_gpus, reduction_devices="gpu", local_proxy_variable=True),
        "uneven_partitioned_ps": lambda: S.UnevenPartitionedPS(reduction_devices="gpu", local_proxy_variable=True),
    }
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=n_gpus), strategy_builder=builders[strategy]())
    # Every process feeds its node's whole batch (batch per GPU x GPUs of the node), as a user of the API does; the
    # remapper keeps this replica's slice, so only that slice crosses PCIe.
    cfg, host_batches = _host_batches(model_name, batch, n_gpus, args.seq)
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values()) // n_gpus
    with ad.scope():
        torch.manual_seed(0)
        if kind == "bert":
            from autodist_b200.models.bert import BertPretrainer
            model = BertPretrainer(cfg)
        elif kind == "lm":
            from autodist_b200.models.lm1b import LM1B
            model = LM1B(cfg)
        else:
            from autodist_b200.models.cnn import ImageClassifier
            model = ImageClassifier(model_name, image_size=224) if model_name == "vgg16" else ImageClassifier(model_name)
        n_params = sum(p.numel() for p in model.parameters())
        phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in host_batches[0].items()}
        loss = model(**phs)
        if kind == "lm":
            opt = torch.optim.Adagrad(model.parameters(), lr=0.2, initial_accumulator_value=1.0)
            train_op = opt.minimize(loss, clip_global_norm=(cfg.max_grad_norm, model.dense_parameters()))
        else:
            opt = torch.optim.Adam(model.parameters(), lr=1e-4) if kind == "bert" else \
                torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
            train_op = opt.minimize(loss)
        sess = ad.create_distributed_session()
        dev = sess.engine.device
        dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches]

        def feed(batches, i):
            b = batches[i % len(batches)]
            return {phs[k]: b[k] for k in phs}

        def step_dev(i):
            sess.run(train_op, feed(dev_batches, i))

        def step_host(i):
            # every step uploads one batch from pinned host memory and reads the loss back; the upload of batch i + 1 is
            # started as soon as step i is launched (the session's `prefetch` argument), so it overlaps the step
            return sess.run([loss, train_op], feed(host_batches, i), prefetch=feed(host_batches, i + 1))[0]

        # this extension's launches inside the device-timed region: eager launches are counted directly, a replayed CUDA graph
        # by the launches of its capture
        counted = {"before": None, "after": None}
        ms, ms_e2e, last, clocks = _timed_with_count(step_dev, step_host, args, world, dev, rank, ops, counted)
        if hasattr(sess.engine, "check_errors"):
            sess.engine.check_errors()
        engine_name = type(sess.engine).__name__
        if getattr(args, "flights", None) and hasattr(sess.engine, "flight_report"):
            _write_flights(args.flights, sess.engine, model_name, strategy, n_gpus, ms / args.steps, rank, world, dev)
        graph_launches = getattr(sess.engine, "graph_kernels", 0)
        eager = (counted["after"] or 0) - (counted["before"] or 0)
        launches = eager if eager > 0 else graph_launches * args.steps
        sess.close()
    del sess, model, opt, dev_batches
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    global_batch = batch * n_gpus
    per_sample = cfg.num_steps if kind == "lm" else 1                 # LM1B counts words: batch x unrolled steps
    unit = {"bert": "sequences/s", "lm": "words/s", "cnn": "images/s"}[kind]
    published = (PUBLISHED_PER_GPU if model_name == "bert-large" else PUBLISHED_RESNET101 if model_name == "resnet101" else {}).get(n_gpus)
    value = global_batch * per_sample * args.steps / (ms / 1e3)
    e2e = global_batch * per_sample * args.steps / (ms_e2e / 1e3)
    conv_own = os.environ.get("AUTODIST_CONV", "own") != "library"
    compute = {"bert": "hand-written sm_100a kernels (tcgen05 GEMM, layernorm, softmax, cross-entropy, Adam)",
               "lm": "tcgen05 GEMM + own LSTM-cell / gather kernels, autograd glue",
               "cnn": ("tcgen05 implicit-GEMM convolutions (forward, dgrad, wgrad)" if conv_own else "library convolutions") +
                      " + own batch-norm / ReLU / max-pool kernels + tcgen05 GEMM for fully connected layers"}[kind]
    return {
        "metric": METRIC.get(kind, f"{model_name} ImageNet-shape training images/sec, max over ranks"),
        "value": round(value, 2), "unit": unit, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / (published * n_gpus), 2) if published else None,
        "dtype": "bf16", "data": DATA[kind],
        "config": {"model": model_name, "parameters": n_params, "global_batch": global_batch,
                   "seq_len": args.seq if kind == "bert" else (cfg.num_steps if kind == "lm" else None),
                   "max_predictions": MAX_PRED if kind == "bert" else None,
                   "tie_word_embeddings": bool(cfg.tie_word_embeddings) if kind == "bert" else None,
                   "compute": compute, "parallelism": f"dp{n_gpus}", "strategy": strategy,
                   "optimizer": {"bert": "Adam, fp32 master + bf16 compute", "lm": "Adagrad 0.2, LSTM gradients clipped at norm 10",
                                 "cnn": "SGD momentum 0.9, fp32 master + bf16 autocast"}[kind],
                   "comm": os.environ.get("AUTODIST_COMM", "fused"),
                   "cuda_graph": os.environ.get("AUTODIST_CUDA_GRAPH", "1") != "0",
                   "l2": "per-step working set (activations + weights > 4 GB) is far larger than the 126 MB L2",
                   "engine": engine_name},
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": unit, "ms_per_step": round(ms_e2e / args.steps, 3),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": last},
        "gpu_launches": int(launches),
        "impl": "ours",
    }


def _write_flights(path, engine, model_name, strategy, n_gpus, ms_step, rank, world, dev):
    """Table of the last step's flights: range, bytes, start since the step's first kernel, duration (max over ranks)."""
    import torch
    rows = engine.flight_report()
    t = torch.tensor([[r[2], r[3]] for r in rows] or [[0.0, 0.0]], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return
    t = t.cpu().tolist()
    lines = [f"# Gradient flights of one {model_name} step, {n_gpus} GPU(s), strategy {strategy}", "",
             f"Eager launches (timed events cannot be captured), {ms_step:.2f} ms per step in this mode. `start` is measured from the",
             "first kernel of the step; `ms` is how long the flight's kernels (collective + optimizer update) held the",
             "communication stream, max over ranks; `GB/s` is the bus bandwidth 2(N-1)/N x bytes / ms of an all-reduce of that",
             "size (the optimizer update is inside the same interval, so this is a lower bound).", "",
             "| flight | elements | MB (fp32) | start ms | ms | bus GB/s |", "|---|---|---|---|---|---|"]
    total = 0.0
    for i, (r, (start, ms)) in enumerate(zip(rows, t)):
        n = r[1] - r[0]
        bus = 2 * (n_gpus - 1) / n_gpus * n * 4 / (ms * 1e-3) / 1e9 if ms > 0 and n_gpus > 1 else 0.0
        total += ms
        lines.append(f"| {i} | {n} | {n * 4 / 2**20:.1f} | {start:.2f} | {ms:.3f} | {bus:.0f} |")
    last_end = max((s + m for s, m in t), default=0.0)
    lines += ["", f"Communication stream busy {total:.2f} ms of the {ms_step:.2f} ms step; the last flight ends {last_end:.2f} ms after the step's first kernel."]
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


def _timed_with_count(step_dev, step_host, args, world, dev, rank, ops, counted):
    """``_timed`` with the extension's launch counter read around the device-timed region only."""
    state = {"n": 0}
    total_warm = args.warmup + 3

    def dev_step(i):
        if state["n"] == total_warm:
            counted["before"] = ops.launch_count
        step_dev(i)
        state["n"] += 1
        if state["n"] == total_warm + args.steps:
            counted["after"] = ops.launch_count

    return _timed(dev_step, step_host, args.steps, args.warmup, world, dev, sampler_rank0=(rank == 0))


def run_library(model_name, args, n_gpus, world, rank):
    """The same measurement for the stock-PyTorch build of the model (cuBLAS / cuDNN / fused attention, torch optimizers, DDP)."""
    import torch
    import torch.distributed as dist
    from baseline import library_models as L

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    kind = _kind(model_name)
    batch = args.batch or _default_batch(model_name)
    torch.manual_seed(0)
    model, opt, cfg = L.build(model_name, dev)
    n_params = L.param_count(model)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True) if world > 1 else model
    _, host_all = _host_batches(model_name, batch, n_gpus, args.seq)
    # this rank's slice of the node batch, still in pinned host memory
    host_batches = [{k: v[rank * batch:(rank + 1) * batch].clone().pin_memory() for k, v in b.items()} for b in host_all]
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches]

    def one(b):
        if kind == "cnn":
            b = dict(b, images=b["images"].contiguous(memory_format=torch.channels_last))
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(**b)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    def step_dev(i):
        one(dev_batches[i % len(dev_batches)])

    def step_host(i):
        b = {k: v.to(dev, non_blocking=True) for k, v in host_batches[i % len(host_batches)].items()}
        return float(one(b).item())

    ms, ms_e2e, last, clocks = _timed(step_dev, step_host, args.steps, args.warmup, world, dev, sampler_rank0=(rank == 0))
    del net, model, opt, dev_batches
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    global_batch = batch * n_gpus
    unit = "sequences/s" if kind == "bert" else "images/s"
    value = global_batch * args.steps / (ms / 1e3)
    e2e = global_batch * args.steps / (ms_e2e / 1e3)
    return {
        "metric": METRIC.get(kind, f"{model_name} ImageNet-shape training images/sec, max over ranks"),
        "value": round(value, 2), "unit": unit, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": DATA[kind],
        "config": {"model": model_name, "parameters": n_params, "global_batch": global_batch, "seq_len": args.seq if kind == "bert" else None,
                   "compute": "stock PyTorch: cuBLAS linears, fused scaled_dot_product_attention, library layernorm, Adam(fused=True)"
                   if kind == "bert" else "stock PyTorch: cuDNN convolutions / batch-norm, channels-last, SGD(foreach=True)",
                   "parallelism": f"dp{n_gpus}", "strategy": "DistributedDataParallel (NCCL)" if world > 1 else "single process",
                   "optimizer": "fp32 master weights, bf16 autocast", "cuda_graph": False},
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": unit, "ms_per_step": round(ms_e2e / args.steps, 3), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4, "last_loss": last},
        "gpu_launches": 0,
        "impl": "library",
    }


_RESULT_FD = None


def _own_stdout():
    """The result line must be the only thing on stdout, but libraries write there too (NCCL prints its version banner
    when its first communicator comes up): point file descriptor 1 at stderr for the rest of the process and keep the
    original for `_emit`."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(record):
    line = (json.dumps(record) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "library", "reference"])
    ap.add_argument("--model", default="bert-large", choices=["bert-large", "bert-base", "bert-tiny", "resnet101", "vgg16",
                                                              "resnet50", "densenet121", "inceptionv3", "lm1b", "lm1b-tiny"])
    ap.add_argument("--strategy", default=None, choices=["allreduce", "allreduce_ef", "powersgd", "parallax", "ps", "partitioned_ps",
                                                         "uneven_partitioned_ps"],
                    help="default: parallax for BERT and LM1B on more than one GPU (dense gradients all-reduced, embedding tables "
                         "through the sparse parameter-server path), allreduce otherwise")
    ap.add_argument("--batch", type=int, default=0, help="samples per GPU (default: 32 sequences, 64 images, 32 for vgg16)")
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--comm", default=None, help="fused (own kernels) or nccl (baseline)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--only", action="store_true", help="measure --model alone: no ResNet-101 block, no library block")
    ap.add_argument("--flights", default=None, metavar="PATH",
                    help="also time every gradient flight of the last step with CUDA events (the step then runs as eager launches, "
                         "not as a CUDA graph) and write the table to PATH; implies --only")
    args = ap.parse_args()
    _own_stdout()
    if args.impl == "reference":
        return reference_arm(args)
    if args.comm:
        os.environ["AUTODIST_COMM"] = args.comm
    if args.no_graph:
        os.environ["AUTODIST_CUDA_GRAPH"] = "0"
    if args.flights:
        os.environ["AUTODIST_FLIGHT_TIMING"] = "1"
        args.only = True
    os.environ.setdefault("AUTODIST_MIN_LOG_LEVEL", "WARNING")
    os.environ.setdefault("AUTODIST_FETCH_MODE", "local")
    args.warmup = max(args.warmup, 3)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    n_gpus = world if world > 1 else args.gpus

    if args.impl == "library":
        out = run_library(args.model, args, n_gpus, world, rank)
        if rank == 0:
            _emit(out)
        return 0

    out = run_ours(args.model, args, n_gpus, world, rank)
    full = args.model == "bert-large" and not args.only and args.batch == 0 and args.strategy is None
    if full:
        # the second half of the headline metric and the same-box library build of both halves, measured in this call
        extra_args = argparse.Namespace(**vars(args))
        extra_args.steps, extra_args.warmup = max(5, args.steps // 2), 3
        try:
            rn = run_ours("resnet101", extra_args, n_gpus, world, rank)
            out["resnet101"] = {k: rn[k] for k in ("metric", "value", "unit", "ms_per_step", "vs_baseline", "e2e", "gpu_launches", "steps", "warmup")}
            out["resnet101"]["config"] = rn["config"]
        except Exception as e:  # the main line must survive a failure of the extra measurements
            out["resnet101"] = {"error": repr(e)[:300]}
        lib = {}
        for name in ("bert-large", "resnet101"):
            try:
                r = run_library(name, extra_args, n_gpus, world, rank)
                lib[name] = {"value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"], "e2e_value": r["e2e"]["value"],
                             "steps": r["steps"], "compute": r["config"]["compute"]}
            except Exception as e:
                lib[name] = {"error": repr(e)[:300]}
        out["library"] = lib
        if "value" in lib.get("bert-large", {}):
            out["vs_library"] = {"value": round(out["value"] / lib["bert-large"]["value"], 3),
                                 "e2e": round(out["e2e"]["value"] / lib["bert-large"]["e2e_value"], 3)}
        if "value" in lib.get("resnet101", {}) and "value" in out.get("resnet101", {}):
            out["resnet101"]["vs_library"] = {"value": round(out["resnet101"]["value"] / lib["resnet101"]["value"], 3),
                                              "e2e": round(out["resnet101"]["e2e"]["value"] / lib["resnet101"]["e2e_value"], 3)}
    if rank == 0:
        _emit(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
