"""Run every strategy on one case with ``--nproc`` CPU ranks (gloo) and compare with the plain-PyTorch oracle.

Usage: ``python run_matrix.py --case c0 --nproc 2``. The parent starts the ranks (RANK / WORLD_SIZE in
the environment, as an external launcher would); every rank iterates over the strategies and exits
non-zero on the first mismatch.
"""
import argparse
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)


def strategies():
    from autodist_b200.strategy import (PS, AllReduce, Parallax, PartitionedAR, PartitionedPS, PSLoadBalancing,
                                        RandomAxisPartitionAR, UnevenPartitionedPS)
    return {
        "PS": (lambda: PS(), 1e-5),
        "PS_proxy": (lambda: PS(local_proxy_variable=True), 1e-5),
        "PSLoadBalancing_proxy": (lambda: PSLoadBalancing(local_proxy_variable=True), 1e-5),
        "PartitionedPS_proxy": (lambda: PartitionedPS(local_proxy_variable=True), 1e-5),
        "PartitionedPS_owners": (lambda: PartitionedPS(num_shards=2, reduction_devices="gpu"), 1e-5),
        "UnevenPartitionedPS_proxy": (lambda: UnevenPartitionedPS(local_proxy_variable=True), 1e-5),
        "AllReduce_None": (lambda: AllReduce(chunk_size=1, all_reduce_spec="NCCL", compressor="NoneCompressor"), 1e-5),
        "AllReduce_chunk512": (lambda: AllReduce(chunk_size=512), 1e-5),
        "AllReduce_Horovod": (lambda: AllReduce(chunk_size=1, compressor="HorovodCompressor"), 2e-2),
        "AllReduce_HorovodEF": (lambda: AllReduce(chunk_size=2, all_reduce_spec="RING",
                                                  compressor="HorovodCompressorEF"), 2e-2),
        "AllReduce_PowerSGD": (lambda: AllReduce(chunk_size=8, compressor="PowerSGDCompressor"), None),
        "Parallax_proxy": (lambda: Parallax(local_proxy_variable=True), 1e-5),
        "PartitionedAR": (lambda: PartitionedAR(), 1e-5),
        "RandomAxisPartitionAR": (lambda: RandomAxisPartitionAR(chunk_size=4, seed=3), 1e-5),
    }


def run_rank(case, nproc, workdir, only=None):
    import numpy as np
    import torch
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.checkpoint.saver import Saver
    from autodist_b200.resource_spec import ResourceSpec
    import cases

    rank = int(os.environ.get("RANK", "0"))
    ref_state, ref_losses = cases.oracle(case)
    factory, _, data_fn, ph_specs, opt_fn, steps = cases.CASES[case]
    data = data_fn()
    failures = []
    for name, (make, tol) in strategies().items():
        if only and name not in only:
            continue
        _reset_default_autodist()
        ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=nproc), strategy_builder=make())
        with ad.scope():
            torch.manual_seed(7)
            model = factory()
            phs = {k: ad.placeholder(shape, dtype, name=k) for k, (shape, dtype) in ph_specs.items()}
            loss = model(**phs)
            opt = opt_fn(list(model.parameters()))
            train_op = opt.minimize(loss)
            saver = Saver()
            sess = ad.create_distributed_session()
            for _ in range(steps):
                lv, _ = sess.run([loss, train_op], feed_dict={phs[k]: data[k] for k in phs})
            state = {n[:-2]: sess.run(n) for n, _ in ad.graph_item.named_parameters()}
            ckpt = saver.save(sess, os.path.join(workdir, f"{case}_{name}", "model"), global_step=steps)
            sess.close()
        worst = 0.0
        for k, ref in ref_state.items():
            got = torch.from_numpy(np.asarray(state[k]))
            worst = max(worst, float((got - ref).abs().max()))
        ok = np.isfinite(worst) and (tol is None or worst <= tol)
        if rank == 0:
            # the checkpoint is a plain state dict under the original names, partitions merged
            plain = torch.load(ckpt, map_location="cpu", weights_only=False)
            fresh = cases.CASES[case][1]()
            fresh.load_state_dict(plain["variables"])
            for k, ref in ref_state.items():
                if tol is not None and float((fresh.state_dict()[k] - ref).abs().max()) > tol:
                    ok = False
        print(f"[rank {rank}] {case} {name}: max|diff|={worst:.3e} tol={tol} {'ok' if ok else 'FAIL'}", flush=True)
        if not ok:
            failures.append(name)
    return failures


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="c0")
    ap.add_argument("--nproc", type=int, default=2)
    ap.add_argument("--only", default="")
    ap.add_argument("--workdir", default="")
    args = ap.parse_args()
    only = [s for s in args.only.split(",") if s]
    if "RANK" in os.environ or args.nproc == 1:
        workdir = args.workdir or tempfile.mkdtemp(prefix="autodist_matrix_")
        failures = run_rank(args.case, args.nproc, workdir, only)
        sys.exit(1 if failures else 0)
    workdir = tempfile.mkdtemp(prefix="autodist_matrix_")
    port = 20000 + (os.getpid() % 20000)
    procs = []
    for r in range(args.nproc):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(args.nproc), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), AUTODIST_PG_TIMEOUT="120")
        procs.append(subprocess.Popen([sys.executable, os.path.abspath(__file__), "--case", args.case, "--nproc",
                                       str(args.nproc), "--only", args.only, "--workdir", workdir], env=env))
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=600))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    sys.exit(0 if all(c == 0 for c in codes) else 1)


if __name__ == "__main__":
    main()
