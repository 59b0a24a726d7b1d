"""Multi-GPU checks of the symmetric-memory kernels (one rank per GPU, started by test_comm_multigpu.py)."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from autodist_b200.parallel.fused_engine import SymmetricArena
    arena = SymmetricArena(dist.group.WORLD, dev, rank, world)
    E = arena.E
    ctx = arena.ctx
    use_mc = os.environ.get("AUTODIST_NVLS", "1") != "0"

    def check(name, got, ref, tol):
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= tol, f"{name}: max err {err} > {tol}"
        if rank == 0:
            print(f"{name}: ok (max err {err:.2e})", flush=True)

    # ---- K1: fp32 in-place all-reduce (peer loads/stores, then through the multicast address if there is one)
    n = 1 << 20
    buf, ptrs, mc = arena.alloc(n, torch.float32)
    for label, mcast in (("p2p", 0), ("nvls", mc)):
        if label == "nvls" and (not mc or not use_mc):
            continue
        torch.manual_seed(100 + rank)
        x = torch.randn(n, device=dev)
        buf.copy_(x)
        ref = x.clone()
        dist.all_reduce(ref)
        ref /= world
        torch.cuda.synchronize(); dist.barrier()
        E.allreduce(*ctx(), ptrs, mcast, 0, n, None, None, None, 1.0 / world, 0)
        torch.cuda.synchronize()
        arena.check()
        check(f"allreduce fp32 {label}", buf, ref, 1e-5)
        dist.barrier()
    # odd sub-range of the buffer (a flight): offsets in elements, multiple of 4
    lo, hi = 4 * 1001, 4 * 50021
    torch.manual_seed(200 + rank)
    x = torch.randn(n, device=dev)
    buf.copy_(x)
    ref = x.clone()
    r = ref[lo:hi].clone(); dist.all_reduce(r); ref[lo:hi] = r / world
    torch.cuda.synchronize(); dist.barrier()
    E.allreduce(*ctx(), ptrs + lo * 4, 0, 0, hi - lo, None, None, None, 1.0 / world, 0)
    torch.cuda.synchronize()
    check("allreduce fp32 sub-range", buf, ref, 1e-5)
    dist.barrier()

    # ---- K1 + K6/K7: 16-bit wire with error feedback, result widened back into the gradient buffer
    for wire_dtype, code in ((torch.bfloat16, 1), (torch.float16, 2)):
        wire, wptrs, wmc = arena.alloc(n, wire_dtype)
        for label, mcast in (("p2p", 0), ("nvls", wmc)):
            if label == "nvls" and (not wmc or not use_mc):
                continue
            torch.manual_seed(300 + rank)
            g = torch.randn(n, device=dev) * 0.01
            res = torch.randn(n, device=dev) * 1e-4
            t = g + res
            c = t.to(wire_dtype)
            ref_res = t - c.float()
            gathered = [torch.empty_like(c) for _ in range(world)]
            dist.all_gather(gathered, c)
            ref = (sum(x.float() for x in gathered) / world).to(wire_dtype).float()
            gg, rr = g.clone(), res.clone()
            torch.cuda.synchronize(); dist.barrier()
            E.allreduce(*ctx(), wptrs, mcast, code, n, gg, rr, gg, 1.0 / world, 0)
            torch.cuda.synchronize()
            arena.check()
            check(f"allreduce {wire_dtype} EF {label} value", gg, ref,
                  (5e-4 if wire_dtype is torch.bfloat16 else 5e-5) if label == "nvls" else (2e-4 if wire_dtype is torch.bfloat16 else 2e-5))
            check(f"allreduce {wire_dtype} EF {label} residual", rr, ref_res, 1e-7)
            dist.barrier()

    # ---- K2: reduce-scatter + Adam on the owner + parameter write to every peer
    # (peer loads / stores first, then the same through the multicast addresses where the fabric has them)
    total = 8192
    grads, gptrs, g_mc = arena.alloc(total, torch.float32)
    p16, p16ptrs, p16_mc = arena.alloc(total, torch.bfloat16)
    p32, p32ptrs, p32_mc = arena.alloc(total, torch.float32)
    for label, mcs in (("p2p", (0, 0, 0)), ("nvls", (g_mc, p16_mc, p32_mc))):
        if label == "nvls" and (not all(mcs) or not use_mc):
            continue
        p16.zero_(); p32.zero_()
        torch.manual_seed(7)
        init = torch.randn(total, device=dev)
        # three segments with round-robin owners: [0,2048) -> 0, [2048, 5000+120) -> 1 % world, rest -> 2 % world
        bounds = [0, 2048, 5120, total]
        owners = [0, 1 % world, 2 % world]
        mine = [(bounds[i], bounds[i + 1]) for i in range(3) if owners[i] == rank]
        n_owned = sum(b - a for a, b in mine)
        master = torch.zeros(max(n_owned, 4), device=dev)
        m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
        seg_start, seg_len, seg_state, prefix, off = [], [], [], [0], 0
        for a, b in mine:
            seg_start.append(a); seg_len.append(b - a); seg_state.append(off)
            master[off:off + b - a] = init[a:b]
            off += b - a
            prefix.append(off)
        if not mine:
            seg_start, seg_len, seg_state, prefix = [0], [0], [0], [0, 0]
        i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)   # noqa: E731
        ref_p = init.clone().requires_grad_(True)
        opt = torch.optim.Adam([ref_p], lr=1e-2)
        lr = torch.tensor([1e-2], device=dev)
        step = torch.zeros(1, dtype=torch.int64, device=dev)
        for it in range(3):
            torch.manual_seed(1000 * it + rank)
            g = torch.randn(total, device=dev)
            grads.copy_(g)
            mean = g.clone(); dist.all_reduce(mean); mean /= world
            ref_p.grad = mean
            opt.step()
            E.increment(step)
            torch.cuda.synchronize(); dist.barrier()
            E.reduce_scatter_update(*ctx(), gptrs, p16ptrs, p32ptrs, mcs[0], mcs[1], mcs[2], master, m1, m2, i64(seg_start), i64(seg_len), i64(seg_state),
                                    None, i64(prefix), 1, lr, step, 0.9, 0.999, 1e-8, 0.0, 0.0, 1.0, False, False, 1.0 / world, 8)
            torch.cuda.synchronize()
            arena.check()
            dist.barrier()
        check(f"reduce_scatter_update {label} fp32 params on every rank", p32, ref_p.detach(), 1e-5)
        check(f"reduce_scatter_update {label} bf16 params on every rank", p16, ref_p.detach(), 2e-2)

    # ---- K4 / K5: sparse rows to / from the owner shards (uneven split of V rows)
    V, H = 1003, 64
    q, rem = divmod(V, world)
    my_rows = q + (1 if rank < rem else 0)
    my_off = rank * q + min(rank, rem)
    cap = q + 1
    shard32, s32ptrs, _ = arena.alloc(cap * H, torch.float32)
    shard16, s16ptrs, _ = arena.alloc(cap * H, torch.bfloat16)
    torch.manual_seed(11)
    table = torch.randn(V, H, device=dev).to(torch.bfloat16)
    shard16.zero_()
    shard16[:my_rows * H].copy_(table[my_off:my_off + my_rows].reshape(-1))
    torch.manual_seed(500 + rank)
    ids = torch.randint(0, V, (777 + 13 * rank,), device=dev)
    out = torch.empty(ids.numel(), H, dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize(); dist.barrier()
    E.embedding_gather_peers(*ctx(), s16ptrs, ids, out, V, 3, 16)
    torch.cuda.synchronize()
    arena.check()
    assert torch.equal(out, table[ids]), "peer gather mismatch"
    if rank == 0:
        print("embedding_gather_peers: ok", flush=True)
    vals = torch.randn(ids.numel(), H, device=dev).to(torch.bfloat16)
    dense = torch.zeros(V, H, device=dev).index_add_(0, ids, vals.float())
    dist.all_reduce(dense)
    dense /= world
    shard32.zero_()
    torch.cuda.synchronize(); dist.barrier()
    E.sparse_scatter_add(*ctx(), s32ptrs, None, ids, vals, V, 1.0 / world, 3, 16)
    torch.cuda.synchronize()
    arena.check()
    check("sparse_scatter_add owner shard", shard32[:my_rows * H].view(my_rows, H), dense[my_off:my_off + my_rows], 1e-4)
    dist.barrier()

    # ---- K3: weight rows sharded over the ranks, gathered tile by tile inside the consuming GEMM
    rows_per, Kd, Md = 256, 512, 384
    wshard, wptrs, _ = arena.alloc(rows_per * Kd, torch.bfloat16)
    torch.manual_seed(21)
    w_full = (torch.randn(rows_per * world, Kd, device=dev) * 0.1).to(torch.bfloat16)
    wshard.copy_(w_full[rank * rows_per:(rank + 1) * rows_per].reshape(-1))
    xin = (torch.randn(Md, Kd, device=dev) * 0.5).to(torch.bfloat16)
    bias = torch.randn(rows_per * world, device=dev)
    yout = torch.empty(Md, rows_per * world, dtype=torch.bfloat16, device=dev)
    gerr = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize(); dist.barrier()
    E.sym_barrier(*ctx(), 1)                       # every owner's shard is in place
    E.gemm_gathered_b(xin, [int(p) for p in wptrs.tolist()], rows_per, yout, 1, bias, gerr, 0)
    E.sym_barrier(*ctx(), 1)                       # nobody overwrites a shard that a peer still reads
    torch.cuda.synchronize()
    arena.check()
    assert gerr.item() == 0
    check("all-gather fused into the GEMM (peer TMA tiles)", yout, xin.float() @ w_full.float().t() + bias, 3e-2)
    dist.barrier()

    # ---- K20: a wait that nothing answers runs out, reports a status, and the context stays usable
    arena.timeout_s = 0.5
    if rank == 0:
        E.sym_barrier(*arena.ctx(), 1)
        torch.cuda.synchronize()
        code = int(arena.error.item())
        assert code >= 100, code
        arena.error.zero_()
        print(f"bounded wait gave up with status {code}: ok", flush=True)
    dist.barrier()
    if rank != 0:
        E.sym_barrier(*arena.ctx(), 1)       # meets rank 0's earlier signal at once; epochs are level again
        torch.cuda.synchronize()
        assert int(arena.error.item()) == 0
    dist.barrier()
    arena.timeout_s = 20.0
    E.sym_barrier(*arena.ctx(), 4)
    torch.cuda.synchronize()
    arena.check()
    dist.barrier()

    # ---- K20: bounded-staleness gate. Every rank publishes its step into every peer's clock row and may proceed while it
    # is at most `staleness` steps ahead of the slowest peer; a rank that would have to wait longer than the limit gets
    # status 200 + (the peer it waited for) and its context stays usable.
    clocks, cptrs, _ = arena.alloc(8, torch.int32)
    clocks.zero_()
    torch.cuda.synchronize(); dist.barrier()
    E.staleness_gate(*arena.ctx(), cptrs, 1, 0, None, None)          # all at step 1: nobody is ahead
    torch.cuda.synchronize()
    arena.check()
    dist.barrier()
    arena.timeout_s = 0.5
    if rank == 0:
        E.staleness_gate(*arena.ctx(), cptrs, 4, 2, None, None)      # three steps ahead of peers that stay at step 1: must give up
        torch.cuda.synchronize()
        code = int(arena.error.item())
        assert 200 < code < 200 + world, code
        arena.error.zero_()
        print(f"staleness gate gave up with status {code} (peer {code - 200} is behind): ok", flush=True)
    dist.barrier()
    if rank != 0:
        E.staleness_gate(*arena.ctx(), cptrs, 3, 2, None, None)      # the others catch up to step 3
        torch.cuda.synchronize()
        assert int(arena.error.item()) == 0
    dist.barrier()
    if rank == 0:
        E.staleness_gate(*arena.ctx(), cptrs, 4, 2, None, None)      # one step ahead now: the gate opens at once
        torch.cuda.synchronize()
        assert int(arena.error.item()) == 0
        print("staleness gate opens once the peers caught up: ok", flush=True)
    arena.timeout_s = 20.0
    dist.barrier()
    arena.check_canaries()                         # no kernel of this rank or a peer wrote outside a symmetric buffer
    y = torch.ones(4, device=dev)
    dist.all_reduce(y)
    assert y[0].item() == world
    if rank == 0:
        print("ALL COMM CHECKS PASSED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
