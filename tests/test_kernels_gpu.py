"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 restatements of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    from autodist_b200 import ops
    return ops.ext(required=True)


@pytest.fixture()
def err():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _check(out, ref, tol, fro=None):
    """Max-norm bound relative to the largest reference value, plus a relative Frobenius bound (default: the same
    tolerance) so that one wrong tile of a large product cannot hide under a loose element-wise bound."""
    ref = ref.float()
    diff = (out.float() - ref).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert diff <= bound, f"max diff {diff} > {bound}"
    denom = ref.norm().item()
    if denom > 0 and out.numel() >= 64:
        rel = ((out.float() - ref).norm().item()) / denom
        assert rel <= (tol if fro is None else fro), f"relative Frobenius error {rel} > {tol if fro is None else fro}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (200, 300, 136), (4096, 1024, 1024), (32, 2, 1024),
                                   (640, 1000, 1024)])
def test_gemm_kmajor(E, err, M, N, K):
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    E.gemm(a, b, c, False, False, 0, None, None, None, 1.0, 0.0, err, 0)
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(c, a.float() @ b.float().t(), 1e-2)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths_fp32_out(E, err, bn):
    torch.manual_seed(1)
    M, N, K = 384, 512, 320
    a, b = _rand(M, K), _rand(N, K)
    c = torch.empty(M, N, dtype=torch.float32, device="cuda")
    E.gemm(a, b, c, False, False, 0, None, None, None, 0.5, 0.0, err, bn)
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(c, 0.5 * (a.float() @ b.float().t()), 2e-3)
    c2 = c.clone()
    E.gemm(a, b, c2, False, False, 0, None, None, None, 0.5, 1.0, err, bn)     # accumulate into fp32
    torch.cuda.synchronize()
    _check(c2, 2 * c, 2e-3)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,batch", [(256, 256, 64, 1), (512, 768, 1024, 1), (304, 520, 200, 1), (1000, 264, 72, 1), (4096, 1024, 2048, 1),
                                         (384, 512, 128, 3)])
def test_gemm_on_sm_pairs(E, err, a_mn, b_mn, M, N, K, batch):
    """The two-CTA kernel (tcgen05.mma.cta_group::2, 256 x 256 tiles, bn = 512): every operand layout, ragged extents
    (rows and columns past the last full tile are zero-filled by TMA and masked in the epilogue), batches, fp32
    accumulation into the output and the bias + GELU epilogue."""
    torch.manual_seed(6)
    a = _rand(batch, K, M) if a_mn else _rand(batch, M, K)
    b = _rand(batch, K, N) if b_mn else _rand(batch, N, K)
    A = a.float().transpose(1, 2) if a_mn else a.float()
    B = b.float() if b_mn else b.float().transpose(1, 2)
    ref = A @ B
    c = torch.empty(batch, M, N, dtype=torch.bfloat16, device="cuda")
    E.gemm(a, b, c, a_mn, b_mn, 0, None, None, None, 1.0, 0.0, err, 512)
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(c, ref, 1e-2)
    c32 = torch.ones(batch, M, N, dtype=torch.float32, device="cuda")
    E.gemm(a, b, c32, a_mn, b_mn, 0, None, None, None, 0.5, 1.0, err, 512)
    bias = torch.randn(N, device="cuda")
    pre, act = torch.empty_like(c), torch.empty_like(c)
    E.gemm(a, b, pre, a_mn, b_mn, 2, bias, act, None, 0.1, 0.0, err, 512)
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(c32, 1.0 + 0.5 * ref, 2e-3)
    _check(pre, 0.1 * ref + bias, 1e-2)
    _check(act, torch.nn.functional.gelu(pre.float(), approximate="tanh"), 1e-2)


def test_gemm_picks_the_pair_kernel_for_large_products_and_matches_the_one_cta_kernel(E, err):
    torch.manual_seed(7)
    M, N, K = 2560, 2304, 512
    a, b = _rand(M, K), _rand(N, K)
    c0, c1 = (torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    E.gemm(a, b, c0, False, False, 0, None, None, None, 1.0, 0.0, err, 0)        # chooser: 90 pair tiles >= 74 pairs
    E.gemm(a, b, c1, False, False, 0, None, None, None, 1.0, 0.0, err, 256)
    torch.cuda.synchronize()
    assert err.item() == 0
    assert torch.equal(c0, c1)          # same products in the same K order: the accumulators agree bit for bit


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 320, 192), (1024, 4096, 4096)])
def test_gemm_mn_major(E, err, a_mn, b_mn, M, N, K):
    """The layouts of the backward GEMMs: dX = dY.W (B is MN-major), dW = dY^T.X (both MN-major)."""
    torch.manual_seed(2)
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    c = torch.empty(M, N, dtype=torch.float32, device="cuda")
    E.gemm(a, b, c, a_mn, b_mn, 0, None, None, None, 1.0, 0.0, err, 0)
    torch.cuda.synchronize()
    assert err.item() == 0
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    _check(c, A @ B.t(), 2e-3)


def test_gemm_epilogues(E, err):
    torch.manual_seed(3)
    M, N, K = 256, 512, 256
    a, b = _rand(M, K, scale=0.2), _rand(N, K, scale=0.2)
    bias = torch.randn(N, device="cuda")
    pre = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    act = torch.empty_like(pre)
    E.gemm(a, b, pre, False, False, 2, bias, act, None, 1.0, 0.0, err, 0)
    ref = a.float() @ b.float().t() + bias
    _check(pre, ref, 1e-2)
    _check(act, torch.nn.functional.gelu(pre.float(), approximate="tanh"), 1e-2)
    # dU = (dG . W) * gelu'(u)
    dg, w = _rand(M, K, scale=0.2), _rand(K, N, scale=0.2)      # w is [K, N]: MN-major B for the contraction over K
    du = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    E.gemm(dg, w, du, False, True, 3, None, None, pre, 1.0, 0.0, err, 0)
    u = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(u, approximate="tanh").backward(dg.float() @ w.float())
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(du, u.grad, 1e-2)


def test_gemm_batched_strided_attention_layout(E, err):
    """Q, K, V are strided views into the fused QKV projection output; the context lands in [B*S, heads*D]."""
    torch.manual_seed(4)
    B, S, Hh, D = 2, 128, 4, 64
    qkv = _rand(B * S, 3 * Hh * D, scale=0.5)
    v5 = qkv.view(B, S, 3, Hh, D)
    q, k, v = (v5[:, :, i].permute(0, 2, 1, 3) for i in range(3))       # [B, heads, S, D] views
    scores = torch.empty(B, Hh, S, S, dtype=torch.bfloat16, device="cuda")
    E.gemm(q, k, scores, False, False, 0, None, None, None, 1.0, 0.0, err, 128)
    ref_s = q.float() @ k.float().transpose(-1, -2)
    _check(scores, ref_s, 1e-2)
    p = torch.softmax(ref_s / 8, -1).to(torch.bfloat16)
    ctx = torch.empty(B * S, Hh * D, dtype=torch.bfloat16, device="cuda")
    ctx_view = ctx.view(B, S, Hh, D).permute(0, 2, 1, 3)
    E.gemm(p, v, ctx_view, False, True, 0, None, None, None, 1.0, 0.0, err, 64)       # V is [S_k, D]: MN-major B
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(ctx_view, p.float() @ v.float(), 1e-2)
    # dK = dS^T . Q : both operands MN-major
    ds = _rand(B, Hh, S, S, scale=0.1)
    dk = torch.empty(B, Hh, S, D, dtype=torch.bfloat16, device="cuda")
    E.gemm(ds, q, dk, True, True, 0, None, None, None, 1.0, 0.0, err, 64)
    torch.cuda.synchronize()
    _check(dk, ds.float().transpose(-1, -2) @ q.float(), 1e-2)


@pytest.mark.parametrize("rows,H,p", [(64, 1024, 0.0), (37, 256, 0.0), (4096, 1024, 0.1)])
def test_layernorm(E, rows, H, p):
    torch.manual_seed(5)
    x, res = _rand(rows, H), _rand(rows, H)
    gamma, beta = torch.randn(H, device="cuda"), torch.randn(H, device="cuda")
    z, y = torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    E.ln_fwd(x, res, gamma, beta, z, y, mean, rstd, 1e-12, p, 1234, None)
    if p == 0.0:
        zr = x.float() + res.float()
        _check(z, zr, 1e-2)
    else:
        kept = ((z.float() - res.float()).abs() > 0).float().mean().item()
        assert abs(kept - (1 - p)) < 0.01
    zr = z.float().requires_grad_(True)
    g = gamma.clone().requires_grad_(True)
    b = beta.clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(zr, (H,), g, b, 1e-12)
    _check(y, yr.detach(), 2e-2)
    dy = _rand(rows, H)
    yr.backward(dy.float())
    dz, dx = torch.empty_like(x), torch.empty_like(x)
    part = torch.zeros(E.ln_bwd_part_floats(H), device="cuda")
    dg, db = torch.empty(H, device="cuda"), torch.empty(H, device="cuda")
    dsum = torch.empty(H, device="cuda")
    E.ln_bwd(dy, z, mean, rstd, gamma, None, dz, dx, part, dg, db, p, 1234, None, False, dsum)
    torch.cuda.synchronize()
    _check(dz, zr.grad, 2e-2)
    _check(dg, g.grad, 2e-2)
    _check(db, b.grad, 2e-2)
    assert float(part.abs().max()) == 0.0                     # the scratch is handed back cleared
    # the extra output: column sums of what the kernel hands on (dx with dropout, dz without) = the bias gradient in front
    _check(dsum, (dx if p > 0 else dz).float().sum(0), 1e-3)
    if p > 0:
        # dx is dz with the forward's dropout decisions: every element is either dropped or scaled by 1/(1-p)
        d, full = dx.float(), dz.float() / (1 - p)
        dropped = d == 0
        assert ((d - full).abs()[~dropped] <= 2e-2 * full.abs().clamp(min=1.0)[~dropped]).all()
        assert abs((~dropped).float().mean().item() - (1 - p)) < 0.01
        same = (dropped == ((z.float() - res.float()) == 0)) | (x.float().abs() < 0.05)
        assert same.float().mean().item() > 0.999      # the same decisions as in the forward pass


@pytest.mark.parametrize("pd", [0.0, 0.1])
def test_softmax(E, pd):
    torch.manual_seed(6)
    B, Hh, S = 3, 4, 128
    x = _rand(B, Hh, S, S, scale=3)
    mask = torch.zeros(B, S, device="cuda")
    mask[:, 100:] = -10000.0
    p, pdrop = torch.empty_like(x), torch.empty_like(x)
    E.softmax_fwd(x, mask, p, pdrop, 0.125, pd, 77, None)
    ref = torch.softmax(x.float() * 0.125 + mask[:, None, None, :], -1)
    _check(p, ref, 1e-2)
    dp = _rand(B, Hh, S, S)
    keep = torch.ones_like(ref)
    if pd > 0:
        keep = (pdrop.float() != 0).float() / (1 - pd)
        keep[p.float() == 0] = 1.0 / (1 - pd)
        assert abs((pdrop.float() != 0).float().mean().item() / (p.float() != 0).float().mean().item() - (1 - pd)) < 0.02
    pr = p.float()
    d = dp.float() * (keep if pd > 0 else 1.0)
    ref_ds = 0.125 * pr * (d - (d * pr).sum(-1, keepdim=True))
    E.softmax_bwd(dp, p, 0.125, pd, 77, None)
    torch.cuda.synchronize()
    if pd == 0:
        _check(dp, ref_ds, 2e-2)
    else:
        ok = (p.float() != 0)
        assert ((dp.float() - ref_ds).abs() * ok).max().item() < 5e-2


def test_xent(E):
    torch.manual_seed(7)
    rows, V, ld = 64, 1003, 1008
    logits = _rand(rows, ld, scale=2)
    labels = torch.randint(0, V, (rows,), device="cuda")
    w = (torch.rand(rows, device="cuda") > 0.3).float()
    xr = logits[:, :V].float().requires_grad_(True)
    per = torch.nn.functional.cross_entropy(xr, labels, reduction="none")
    ref = (per * w).sum() / (w.sum() + 1e-5)
    ref.backward()
    denom, loss = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    E.xent(logits, labels, w, denom, loss, V, 1.0, True, 1e-5)
    torch.cuda.synchronize()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    _check(logits[:, :V], xr.grad, 2e-2)
    assert logits[:, V:].abs().max().item() == 0


def test_embedding_and_row_ops(E, err):
    torch.manual_seed(8)
    V, H, B, S = 500, 256, 4, 32
    word, pos, typ = _rand(V, H), _rand(64, H), _rand(2, H)
    ids = torch.randint(0, V, (B * S,), device="cuda")
    tt = torch.randint(0, 2, (B * S,), device="cuda")
    z = torch.empty(B * S, H, dtype=torch.bfloat16, device="cuda")
    E.embed_sum(word, pos, typ, ids, tt, z, S, err)
    assert err.item() == 0
    ref = word.float()[ids] + pos.float()[torch.arange(B * S, device="cuda") % S] + typ.float()[tt]
    _check(z, ref, 1e-2)
    dz = _rand(B * S, H)
    dword = torch.zeros(V, H, device="cuda")
    E.scatter_add_rows(dword, ids, dz, 1.0)
    _check(dword, torch.zeros(V, H, device="cuda").index_add_(0, ids, dz.float()), 1e-3)
    dpos = torch.zeros(S, H, device="cuda")
    E.strided_rowsum(dz, dpos, S, S, B)
    _check(dpos, dz.float().view(B, S, H).sum(0), 1e-3)
    part = torch.empty(E.colsum_parts(B * S) * 2 * H, device="cuda")
    dtyp = torch.zeros(2, H, device="cuda")
    E.keyed_colsum(dz, tt, part, dtyp, 2, False)
    _check(dtyp, torch.zeros(2, H, device="cuda").index_add_(0, tt, dz.float()), 1e-3)
    dbias = torch.zeros(H, device="cuda")
    E.keyed_colsum(dz, None, part, dbias, 1, False)
    _check(dbias, dz.float().sum(0), 1e-3)
    idx = torch.randperm(B * S, device="cuda")[:20]
    out = torch.empty(20, H, dtype=torch.bfloat16, device="cuda")
    E.gather_rows(z, idx, out)
    assert torch.equal(out, z[idx])
    base = z.clone()
    E.scatter_add_rows_bf16(base, idx, out)
    torch.cuda.synchronize()
    exp = z.float()
    exp[idx] += out.float()
    _check(base, exp, 1e-2)


def test_optimizers_match_torch(E):
    torch.manual_seed(9)
    n = 10007
    lr = torch.tensor([1e-2], device="cuda")
    step = torch.zeros(1, dtype=torch.int64, device="cuda")
    for name in ("adam", "sgd", "adagrad"):
        p0 = torch.randn(n, device="cuda")
        ref_p = p0.clone().requires_grad_(True)
        opt = {"adam": lambda: torch.optim.Adam([ref_p], lr=1e-2, weight_decay=0.01),
               "sgd": lambda: torch.optim.SGD([ref_p], lr=1e-2, momentum=0.9, weight_decay=0.01),
               "adagrad": lambda: torch.optim.Adagrad([ref_p], lr=1e-2, eps=1e-10)}[name]()
        p, s1, s2 = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        p16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        step.zero_()
        for _ in range(3):
            g = torch.randn(n, device="cuda")
            ref_p.grad = g.clone()
            opt.step()
            E.increment(step)
            if name == "adam":
                E.adam_update(p, g, s1, s2, p16, lr, 0.9, 0.999, 1e-8, 0.01, False, step, 1.0)
            elif name == "sgd":
                E.sgd_update(p, g, s1, p16, lr, 0.9, 0.0, 0.01, False, step, 1.0)
            else:
                E.adagrad_update(p, g, s1, p16, lr, 1e-10, 0.0, 1.0)
        torch.cuda.synchronize()
        assert (p - ref_p.detach()).abs().max().item() < 1e-5, name
        assert (p16.float() - p).abs().max().item() < 2e-2


def test_functional_linear_matches_torch():
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(10)
    x = (torch.randn(3, 40, 256, device="cuda") * 0.5).requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).requires_grad_(True)
    b = torch.randn(512, device="cuda").requires_grad_(True)
    for act in (None, "gelu"):
        for t in (x, w, b):
            t.grad = None
        y = Fn.linear(x.to(torch.bfloat16), w, b, activation=act)
        dy = torch.randn_like(y.float())
        y.float().backward(dy)
        gx, gw, gb = x.grad.clone(), w.grad.clone(), b.grad.clone()
        for t in (x, w, b):
            t.grad = None
        ref = torch.nn.functional.linear(x, w, b)
        if act == "gelu":
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        ref.backward(dy)
        _check(y, ref.detach(), 2e-2)
        _check(gx, x.grad, 3e-2)
        _check(gw, w.grad, 3e-2)
        _check(gb, b.grad, 3e-2)
    Fn.check_errors()


def test_lstm_cell_and_clip(E):
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(11)
    B, S = 16, 96
    gates = torch.randn(B, 4 * S, device="cuda", requires_grad=True)
    c_prev = torch.randn(B, S, device="cuda", requires_grad=True)
    c, h = Fn.lstm_cell(gates, c_prev, 1.0)
    dh, dc = torch.randn(B, S, device="cuda"), torch.randn(B, S, device="cuda")
    (c * dc).sum().backward(retain_graph=True)
    (h.float() * dh).sum().backward()
    got = (gates.grad.clone(), c_prev.grad.clone())
    gates.grad = c_prev.grad = None
    i, j, f, o = gates.chunk(4, 1)
    c_ref = torch.sigmoid(f + 1.0) * c_prev + torch.sigmoid(i) * torch.tanh(j)
    h_ref = torch.sigmoid(o) * torch.tanh(c_ref)
    ((c_ref * dc).sum() + (h_ref * dh).sum()).backward()
    _check(c, c_ref.detach(), 1e-5)
    _check(h, h_ref.detach(), 1e-2)
    _check(got[0], gates.grad, 1e-2)      # h is rounded to bf16 on the way out; its gradient path is exact
    _check(got[1], c_prev.grad, 1e-2)     # the gradient arriving through the bf16 output h is itself bf16
    gs = [torch.randn(1000, device="cuda") * 3, torch.randn(77, 13, device="cuda")]
    ref_norm = torch.sqrt(sum((g ** 2).sum() for g in gs))
    expect = [g * (5.0 / (ref_norm + 1e-6)) for g in gs]
    Fn.clip_by_global_norm_(gs, 5.0)
    for g, e in zip(gs, expect):
        _check(g, e, 1e-5)
    small = [torch.ones(4, device="cuda") * 0.1]
    Fn.clip_by_global_norm_(small, 5.0)
    assert torch.equal(small[0], torch.ones(4, device="cuda") * 0.1)


def test_power_sgd_kernels_match_the_torch_compressor():
    from autodist_b200.kernel.synchronization.compressor import Compressor
    from autodist_b200.parallel.comm import LocalBackend

    class Bucket:
        def member_shapes(self):
            return [(96, 80), (80,), (33, 7, 5)]

    torch.manual_seed(12)
    flat = torch.randn(96 * 80 + 80 + 33 * 35)
    for rank in (1, 2):
        cpu = Compressor.create("PowerSGDCompressor", Bucket(), rank=rank)
        gpu = Compressor.create("PowerSGDCompressor", Bucket(), rank=rank)
        for step in range(3):
            g = flat * (step + 1)
            a = cpu.reduce(g.clone(), LocalBackend())
            b = gpu.reduce(g.clone().cuda(), LocalBackend())
            _check(b.cpu(), a, 1e-4)
            _check(gpu.error.cpu(), cpu.error, 1e-4)


@pytest.mark.parametrize("pd", [0.0, 0.1])
def test_softmax_fused_into_the_attention_gemms(E, err, pd):
    """QK^T with scale + mask + softmax (+ dropout) in the epilogue, and dP -> dS likewise, against the two-kernel path."""
    torch.manual_seed(14)
    B, Hh, S, D = 2, 3, 128, 64
    q, k, v = _rand(B, Hh, S, D, scale=0.7), _rand(B, Hh, S, D, scale=0.7), _rand(B, Hh, S, D)
    mask = torch.zeros(B, S, device="cuda")
    mask[:, 120:] = -10000.0
    step = torch.full((1,), 3, dtype=torch.int64, device="cuda")
    scores = torch.empty(B, Hh, S, S, dtype=torch.bfloat16, device="cuda")
    p_ref, pd_ref = torch.empty_like(scores), torch.empty_like(scores)
    E.gemm(q, k, scores, False, False, 0, None, None, None, 1.0, 0.0, err, 128)
    E.softmax_fwd(scores, mask, p_ref, pd_ref if pd > 0 else None, 0.125, pd, 99, step)
    p, pdrop = torch.empty_like(scores), torch.empty_like(scores)
    E.gemm_softmax(q, k, p, pdrop if pd > 0 else None, mask, None, False, 0.125, pd, 99, step, err)
    exact = torch.softmax((q.float() @ k.float().transpose(-1, -2)) * 0.125 + mask[:, None, None, :], -1)
    _check(p, exact, 1e-2)                      # the fused form never rounds the scores to bf16
    _check(p, p_ref.float(), 2e-2)
    if pd > 0:
        assert torch.equal(pdrop == 0, pd_ref == 0)          # the same dropout decisions as the stand-alone kernel
    dctx = _rand(B, Hh, S, D, scale=0.3)
    ds_ref = torch.empty_like(scores)
    E.gemm(dctx, v, ds_ref, False, False, 0, None, None, None, 1.0, 0.0, err, 128)
    E.softmax_bwd(ds_ref, p, 0.125, pd, 99, step)
    ds = torch.empty_like(scores)
    E.gemm_softmax(dctx, v, ds, None, None, p, True, 0.125, pd, 99, step, err)
    torch.cuda.synchronize()
    assert err.item() == 0
    _check(ds, ds_ref.float(), 3e-2)


def _rel_fro(out, ref):
    return ((out.float() - ref).norm() / ref.norm().clamp_min(1e-12)).item()


# (N, Cin, H, W, Cout, k, stride, pad): the filter shapes of ResNet-101 (3x3/s1, 3x3/s2, 1x1, 1x1/s2), odd image sizes,
# channel counts below one 64-channel block, and outputs wider than one N tile
CONV_CASES = [(3, 16, 13, 15, 24, 3, 1, 1), (4, 64, 14, 14, 64, 3, 1, 1), (2, 128, 28, 28, 128, 3, 2, 1), (3, 64, 9, 11, 256, 1, 1, 0),
              (2, 256, 14, 14, 512, 1, 2, 0), (2, 72, 7, 7, 320, 3, 1, 1), (5, 32, 17, 9, 48, 3, 2, 1), (2, 64, 8, 8, 64, 3, 1, 0),
              (8, 512, 7, 7, 512, 3, 1, 1), (2, 40, 12, 12, 40, 5, 1, 2), (2, 24, 11, 13, 32, 3, 2, 0)]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CONV_CASES)
def test_implicit_gemm_convolution_matches_the_library(n, cin, h, w, cout, k, stride, pad):
    """Forward, input gradient and weight gradient of the tcgen05 implicit-GEMM convolution against ``F.conv2d`` in fp32."""
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(15)
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).float().to(memory_format=torch.channels_last).requires_grad_(True)
    wt = (torch.randn(cout, k, k, cin, device="cuda") / math.sqrt(cin * k * k)).to(torch.bfloat16).float().requires_grad_(True)
    b = torch.randn(cout, device="cuda").requires_grad_(True)
    y = Fn.conv2d(x.to(torch.bfloat16), wt, b, stride, pad)
    dy = torch.randn_like(y.float()).to(torch.bfloat16).float()
    y.float().backward(dy)
    gx, gw, gb = x.grad.clone(), wt.grad.clone(), b.grad.clone()
    x.grad = wt.grad = b.grad = None
    ref = torch.nn.functional.conv2d(x, wt.permute(0, 3, 1, 2), b, stride, pad)
    ref.backward(dy)
    Fn.check_errors()
    assert y.shape == ref.shape
    _check(y, ref.detach(), 1e-2)
    assert _rel_fro(y, ref.detach()) < 2 ** -8
    _check(gx, x.grad, 1e-2)
    assert _rel_fro(gx, x.grad) < 2 ** -7           # dx is rounded to bf16 once
    _check(gw, wt.grad, 2e-3)
    assert _rel_fro(gw, wt.grad) < 1e-3             # fp32 accumulation and fp32 output
    _check(gb, b.grad, 2e-3)


@pytest.mark.parametrize("n,h,w,cout,k,stride,pad", [(2, 224, 224, 64, 7, 2, 3), (3, 31, 29, 64, 3, 1, 1), (2, 37, 41, 32, 3, 2, 0)])
def test_first_layer_convolution_with_three_input_channels(n, h, w, cout, k, stride, pad):
    """The row-tap path: the image is padded to 8 channels with its halo and each filter row is one 64-element K block."""
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(17)
    x = torch.randn(n, 3, h, w, device="cuda").to(torch.bfloat16).float().to(memory_format=torch.channels_last)
    wt = (torch.randn(cout, k, k, 3, device="cuda") / math.sqrt(3 * k * k)).to(torch.bfloat16).float().requires_grad_(True)
    y = Fn.conv2d(x, wt, None, stride, pad)
    dy = torch.randn_like(y.float()).to(torch.bfloat16).float()
    y.float().backward(dy)
    gw = wt.grad.clone()
    wt.grad = None
    ref = torch.nn.functional.conv2d(x, wt.permute(0, 3, 1, 2), None, stride, pad)
    ref.backward(dy)
    Fn.check_errors()
    assert y.shape == ref.shape
    _check(y, ref.detach(), 1e-2)
    assert _rel_fro(y, ref.detach()) < 2 ** -8
    _check(gw, wt.grad, 2e-3)
    assert _rel_fro(gw, wt.grad) < 1e-3


def test_convolution_epilogue_bias_relu_and_batch_norm_sums():
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(18)
    x = torch.randn(6, 64, 14, 14, device="cuda").to(torch.bfloat16).to(memory_format=torch.channels_last).requires_grad_(True)
    wt = (torch.randn(136, 3, 3, 64, device="cuda") / 24).to(torch.bfloat16).float().requires_grad_(True)
    b = torch.randn(136, device="cuda")
    stats = torch.zeros(2, 136, device="cuda")
    y = Fn.conv2d(x, wt, b, 1, 1, relu=True, stats=stats)
    dy = torch.randn_like(y.float()).to(torch.bfloat16).float()
    y.float().backward(dy)
    gx, gw = x.grad.clone(), wt.grad.clone()
    x.grad = wt.grad = None
    ref = torch.relu(torch.nn.functional.conv2d(x.float(), wt.permute(0, 3, 1, 2), b, 1, 1))
    ref.backward(dy)
    Fn.check_errors()
    _check(y, ref.detach(), 1e-2)
    yf = y.float()
    _check(stats[0], yf.sum((0, 2, 3)), 1e-4)                # the sums are those of the stored (bf16-rounded) output
    _check(stats[1], (yf * yf).sum((0, 2, 3)), 1e-4)
    assert _rel_fro(gx, x.grad.float()) < 2 ** -7
    assert _rel_fro(gw, wt.grad) < 1e-3


@pytest.mark.parametrize("relu", [False, True])
def test_batch_norm_kernels_match_the_library(relu):
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(16)
    x = (torch.randn(6, 32, 9, 11, device="cuda") * 2 + 0.5).to(memory_format=torch.channels_last).requires_grad_(True)
    g = (torch.rand(32, device="cuda") + 0.5).requires_grad_(True)
    b = torch.randn(32, device="cuda").requires_grad_(True)
    rm, rv = torch.zeros(32, device="cuda"), torch.ones(32, device="cuda")
    y = Fn.batch_norm(x.to(torch.bfloat16), g, b, rm, rv, True, 0.1, 1e-5, relu)
    dy = torch.randn_like(y.float())
    y.float().backward(dy)
    got = (x.grad.clone(), g.grad.clone(), b.grad.clone())
    x.grad = g.grad = b.grad = None
    rm2, rv2 = torch.zeros(32, device="cuda"), torch.ones(32, device="cuda")
    xq = x.detach().to(torch.bfloat16).float().requires_grad_(True)            # the kernels see the bf16-rounded input
    ref = torch.nn.functional.batch_norm(xq, rm2, rv2, g, b, True, 0.1, 1e-5)
    ref = torch.relu(ref) if relu else ref
    ref.backward(dy)
    _check(y, ref.detach(), 2e-2)
    _check(got[0], xq.grad, 3e-2)
    _check(got[1], g.grad, 3e-2)
    _check(got[2], b.grad, 3e-2)
    _check(rm, rm2, 1e-2)
    _check(rv, rv2, 1e-2)


@pytest.mark.parametrize("cin,width,stride", [(64, 16, 1), (32, 16, 2), (32, 16, 1)])
def test_residual_fork_gradient_is_added_inside_the_input_gradient_kernel(cin, width, stride, monkeypatch):
    """A bottleneck block with the fork fusion (the skip path's gradient added in the first convolution's dgrad epilogue)
    against the same block with autograd's own accumulation, and against the fp32 library computation."""
    from autodist_b200.models import cnn
    torch.manual_seed(23)
    block = cnn.Bottleneck(cin, width, stride).cuda().train()
    x0 = torch.randn(4, cin, 14, 14, device="cuda").to(torch.bfloat16).to(memory_format=torch.channels_last)
    grads = {}
    for mode in (True, False):
        monkeypatch.setattr(cnn, "FORK_FUSION", mode)
        x = x0.clone().requires_grad_(True)
        xin = x * 1.0                                         # a non-leaf input, as inside a network
        y = block(xin)
        torch.manual_seed(5)
        dy = torch.randn_like(y)
        block.zero_grad()
        y.backward(dy)
        grads[mode] = (y.detach().float(), x.grad.float().clone(), block.a.conv.weight.grad.float().clone())
    for a, b in zip(grads[True], grads[False]):
        _check(a, b, 2e-2)
    # library reference in fp32 on the same (bf16-rounded) input
    monkeypatch.setattr(cnn, "CONV_MODE", "library")
    monkeypatch.setattr(cnn, "NORM_POOL_MODE", "library")
    monkeypatch.setattr(cnn, "FORK_FUSION", False)
    ref = cnn.Bottleneck(cin, width, stride).cuda().train()
    ref.load_state_dict(block.state_dict())
    for m in ref.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            m.reset_running_stats()
    x = x0.float().requires_grad_(True)
    yr = ref(x)
    yr.backward(dy.float())
    _check(grads[True][0], yr.detach(), 5e-2)
    # an activation that bf16 rounding moves across zero flips its ReLU mask, which changes single elements of dx by the
    # size of a gradient: the input gradient is compared in the Frobenius norm only
    rel = ((grads[True][1] - x.grad).norm() / x.grad.norm()).item()
    assert rel < 0.1, rel


@pytest.mark.parametrize("k,stride,pad", [(3, 2, 1), (2, 2, 0)])
def test_max_pool_kernels_match_the_library(k, stride, pad):
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(17)
    x = torch.relu(torch.randn(4, 16, 13, 14, device="cuda")).to(torch.bfloat16).to(memory_format=torch.channels_last)   # many ties at 0
    x = x.float().requires_grad_(True)
    y = Fn.max_pool2d(x.to(torch.bfloat16), k, stride, pad)
    dy = torch.randn_like(y.float())
    y.float().backward(dy)
    gx = x.grad.clone()
    x.grad = None
    ref = torch.nn.functional.max_pool2d(x, k, stride, pad)
    ref.backward(dy.to(torch.bfloat16).float())
    assert torch.equal(y.float(), ref.detach())
    _check(gx, x.grad, 2e-2)


def test_sparse_lookup_matches_embedding_with_sparse_gradient():
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(18)
    table = torch.randn(500, 64, device="cuda", requires_grad=True)
    ids = torch.randint(0, 500, (7, 9), device="cuda")
    ids[0, :4] = 3                                                             # repeated rows accumulate
    out = Fn.sparse_lookup(table, ids)
    assert out.dtype == torch.bfloat16 and out.shape == (7, 9, 64)
    dy = torch.randn(7, 9, 64, device="cuda")
    out.float().backward(dy)
    assert table.grad.is_sparse
    got = table.grad.to_dense()
    table.grad = None
    ref = torch.nn.functional.embedding(ids, table)
    ref.backward(dy.to(torch.bfloat16).float())
    _check(out, ref.detach(), 1e-2)
    _check(got, table.grad, 1e-2)


def test_tail_handling_sweep_of_flat_kernels(E):
    """Every length from 1 to 257 (vector tails, odd and prime sizes) for the kernels that take a flat element count;
    guard words after each output buffer must stay untouched."""
    torch.manual_seed(19)
    lr = torch.tensor([1e-2], device="cuda")
    step = torch.ones(1, dtype=torch.int64, device="cuda")
    guard = 8
    for n in list(range(1, 258)) + [1021, 4099]:
        g = torch.randn(n, device="cuda")
        bufs = [torch.full((n + guard,), 7.0, device="cuda") for _ in range(3)]      # p, m, v each followed by guard words
        p, m, v = (b[:n] for b in bufs)                                              # each starts at an aligned base
        p.copy_(torch.randn(n, device="cuda"))
        m.zero_()
        v.zero_()
        p16 = torch.full((n + guard,), 7.0, dtype=torch.bfloat16, device="cuda")
        ref = p.clone().requires_grad_(True)
        opt = torch.optim.Adam([ref], lr=1e-2)
        ref.grad = g.clone()
        opt.step()
        E.adam_update(p, g, m, v, p16[:n], lr, 0.9, 0.999, 1e-8, 0.0, False, step, 1.0)
        assert (p - ref.detach()).abs().max().item() < 1e-5, n
        assert (p16[:n].float() - p).abs().max().item() < 2e-2, n
        assert all((b[n:] == 7.0).all() for b in bufs) and (p16[n:] == 7.0).all(), f"write past the end at n={n}"
    from autodist_b200.ops import functional as Fn
    for n in (1, 2, 3, 7, 31, 33, 255, 257, 1023, 1025):
        gs = [torch.randn(n, device="cuda") * 4]
        norm = gs[0].norm()
        expect = gs[0] * min(1.0, 2.0 / (norm.item() + 1e-6))
        Fn.clip_by_global_norm_(gs, 2.0)
        _check(gs[0], expect, 1e-5)


@pytest.mark.parametrize("rows", [1, 2, 3, 31, 127, 257, 1031])
def test_row_kernels_with_prime_row_counts(E, rows):
    torch.manual_seed(20)
    H = 64
    x = _rand(rows, H)
    # layer-norm forward over an odd number of rows
    gamma, beta = torch.randn(H, device="cuda"), torch.randn(H, device="cuda")
    z, y = torch.empty_like(x), torch.full((rows + 1, H), 7.0, dtype=torch.bfloat16, device="cuda")
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    E.ln_fwd(x, None, gamma, beta, z, y[:rows], mean, rstd, 1e-12, 0.0, 0, None)
    _check(y[:rows], torch.nn.functional.layer_norm(x.float(), (H,), gamma, beta, 1e-12), 2e-2)
    assert (y[rows] == 7.0).all()
    # row gather (bf16 and fp32 tables) with repeated and boundary rows
    table = torch.randn(rows, H, device="cuda")
    ids = torch.randint(0, rows, (rows + 2,), device="cuda")
    ids[0], ids[-1] = 0, rows - 1
    out = torch.full((rows + 3, H), 7.0, dtype=torch.bfloat16, device="cuda")
    E.gather_rows_f32(table, ids, out[:rows + 2])
    _check(out[:rows + 2], table[ids].to(torch.bfloat16).float(), 1e-6)
    assert (out[rows + 2] == 7.0).all()
    E.gather_rows(x, ids, out[:rows + 2])
    assert torch.equal(out[:rows + 2], x[ids]) and (out[rows + 2] == 7.0).all()
    # batch-norm statistics over a prime number of rows
    from autodist_b200.ops import functional as Fn
    xb = x.view(rows, 1, 1, H).permute(0, 3, 1, 2)
    if rows > 1:
        yb = Fn.batch_norm(xb, torch.ones(H, device="cuda"), torch.zeros(H, device="cuda"), None, None, True, 0.1, 1e-5, False)
        ref = torch.nn.functional.batch_norm(xb.float(), None, None, None, None, True, 0.1, 1e-5)
        _check(yb, ref, 3e-2)


@pytest.mark.parametrize("kind", ["sgd", "adagrad", "lazy_adam"])
def test_sparse_row_updates_match_the_torch_sparse_optimizers(kind):
    from autodist_b200.ops import functional as Fn
    torch.manual_seed(21)
    V, H = 301, 40
    p0 = torch.randn(V, H, device="cuda")
    ref = p0.clone().requires_grad_(True)
    opt = {"sgd": lambda: torch.optim.SGD([ref], lr=0.1), "adagrad": lambda: torch.optim.Adagrad([ref], lr=0.1, eps=1e-10),
           "lazy_adam": lambda: torch.optim.SparseAdam([ref], lr=0.01)}[kind]()
    p = p0.clone()
    p16 = p0.to(torch.bfloat16)
    s1, s2 = torch.zeros_like(p), torch.zeros_like(p)
    step = torch.zeros(1, dtype=torch.int64, device="cuda")
    for it in range(4):
        ids = torch.randint(0, V, (64,), device="cuda")
        ids[:8] = 5                                                           # duplicates are summed by the coalesce
        vals = torch.randn(64, H, device="cuda")
        g = torch.sparse_coo_tensor(ids[None], vals, (V, H))
        ref.grad = g
        opt.step()
        step += 1
        Fn.sparse_rows_update_(kind, p, g, 0.01 if kind == "lazy_adam" else 0.1, s1, s2, step, eps=1e-8 if kind == "lazy_adam" else 1e-10,
                               table_bf16=p16)
    torch.cuda.synchronize()
    assert (p - ref.detach()).abs().max().item() < 1e-5
    untouched = torch.ones(V, dtype=torch.bool, device="cuda")
    assert (p16.float() - p).abs().max().item() < 2e-2
    # ids outside the table are ignored
    before = p.clone()
    Fn.sparse_rows_update_("sgd", p, (torch.tensor([V + 3, -1], device="cuda"), torch.ones(2, H, device="cuda")), 0.1)
    torch.cuda.synchronize()
    assert torch.equal(p, before) and untouched.all()
