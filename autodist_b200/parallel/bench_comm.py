"""All-reduce micro-benchmark: the fused symmetric-memory kernel against NCCL, device-timed, max over ranks.

``python -m torch.distributed.run --nproc-per-node N -m autodist_b200.parallel.bench_comm`` prints one JSON line
per message size with time, algorithm bandwidth, bus bandwidth (``2 (N-1)/N * bytes / time``) and the fraction of a
770 GB/s per-direction peer-copy bandwidth (measured on an 8 x B200 NVSwitch box; ``--link-gbs`` overrides it).
"""
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, iters, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def single_rank(n=64 << 20):
    """The communication kernels with a world of one rank (no peer traffic): the form a profiler can capture,
    since a kernel that waits for other ranks is never run under a profiler that serialises launches."""
    from autodist_b200 import ops
    E = ops.ext(required=True)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flags = torch.zeros(E.MAX_COMM_BLOCKS * 8, dtype=torch.int32, device=dev)
    ctx = (torch.tensor([flags.data_ptr()], dtype=torch.int64, device=dev),
           torch.zeros(E.MAX_COMM_BLOCKS + 8, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev), 0, 1, 5.0)
    ptr = lambda t: torch.tensor([t.data_ptr()], dtype=torch.int64, device=dev)   # noqa: E731
    grad = torch.randn(n, device=dev)
    wire = torch.empty(n, dtype=torch.float16, device=dev)
    res = torch.zeros(n, device=dev)
    rows = []
    for label, fn in (
        ("allreduce fp32 in place (1 rank)", lambda: E.allreduce(*ctx, ptr(grad), 0, 0, n, None, None, None, 1.0, 64)),
        ("allreduce fp16 wire + error feedback (1 rank)", lambda: E.allreduce(*ctx, ptr(wire), 0, 2, n, grad, res, grad, 1.0, 64)),
    ):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        rows.append({"kernel": label, "elements": n, "ms": round(s.elapsed_time(e), 4)})
    p16 = torch.empty(n, dtype=torch.bfloat16, device=dev)
    p32 = torch.empty(n, device=dev)
    master, m1, m2 = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)   # noqa: E731
    lr, step = torch.tensor([1e-3], device=dev), torch.ones(1, dtype=torch.int64, device=dev)
    fn = lambda: E.reduce_scatter_update(*ctx, ptr(grad), ptr(p16), ptr(p32), master, m1, m2, i64([0]), i64([n]), i64([0]),   # noqa: E731
                                         i64([0, n]), 1, lr, step, 0.9, 0.999, 1e-8, 0.0, 0.0, 1.0, False, False, 1.0, 64)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    rows.append({"kernel": "reduce_scatter_update Adam (1 rank)", "elements": n, "ms": round(s.elapsed_time(e), 4),
                 "gbs": round(n * 38 / s.elapsed_time(e) / 1e6, 1)})
    assert int(ctx[2].item()) == 0
    for r in rows:
        print(json.dumps(r), flush=True)


def main():
    import sys
    if "--single" in sys.argv:
        return single_rank()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from autodist_b200.parallel.fused_engine import SymmetricArena
    arena = SymmetricArena(dist.group.WORLD, dev, rank, world)
    E = arena.E
    link = 770.0
    if "--link-gbs" in sys.argv:
        link = float(sys.argv[sys.argv.index("--link-gbs") + 1])
    for mib in (1, 16, 64, 256, 1024):
        n = mib * (1 << 20) // 4
        buf, ptrs, mc = arena.alloc(n, torch.float32)
        buf.normal_()
        plain = torch.randn(n, device=dev)
        iters = 20 if mib <= 64 else 5
        row = {"bytes": n * 4, "ranks": world}
        for label, mcast in (("fused_p2p", 0), ("fused_nvls", mc)):
            if label == "fused_nvls" and not mc:
                continue
            for blocks in (32, 64, 128):
                ms = _timed(lambda: E.allreduce(*arena.ctx(), ptrs, mcast, 0, n, None, None, None, 1.0 / world, blocks), iters, world)
                bus = 2 * (world - 1) / world * n * 4 / ms / 1e6
                row[f"{label}_b{blocks}_ms"] = round(ms, 4)
                row[f"{label}_b{blocks}_busbw_gbs"] = round(bus, 1)
        ms = _timed(lambda: dist.all_reduce(plain), iters, world)
        row["nccl_ms"] = round(ms, 4)
        row["nccl_busbw_gbs"] = round(2 * (world - 1) / world * n * 4 / ms / 1e6, 1)
        best = max(v for k, v in row.items() if k.endswith("busbw_gbs") and k.startswith("fused"))
        row["fused_best_frac_of_link"] = round(best / link, 3)
        arena.check()
        if rank == 0:
            print(json.dumps(row), flush=True)
        del buf
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
