"""All-reduce micro-benchmark: the fused symmetric-memory kernel against NCCL, device-timed, max over ranks.

``python -m torch.distributed.run --nproc-per-node N -m autodist_b200.parallel.bench_comm`` prints one JSON line
per message size with time, algorithm bandwidth, bus bandwidth (``2 (N-1)/N * bytes / time``) and the fraction of the
measured 770 GB/s per-direction peer-copy bandwidth of this pool.
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


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from autodist_b200.parallel.fused_engine import SymmetricArena
    arena = SymmetricArena(dist.group.WORLD, dev, rank, world)
    E = arena.E
    link = 770.0
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
