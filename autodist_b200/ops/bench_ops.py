"""Micro-benchmarks of the hand-written kernels against the measured peaks.

``python -m autodist_b200.ops.bench_ops [--json out.json]`` times the tcgen05 GEMM at the shapes of the BERT-large
step (forward, dX and dW layouts) with CUDA events (warm-up, L2 flushed between iterations by streaming a 256 MB
buffer) and reports TFLOP/s next to ``torch.matmul`` (cuBLAS) at the same shape, plus the bandwidth-bound kernels
in GB/s.
"""
import argparse
import json
import os

import torch


def _time(fn, iters=10, flush=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def _cnn_rows(E, dev, flush, hbm):
    """Batch-norm (+ReLU), max-pool, fp32 -> bf16 row gather and the row-sparse Adagrad update, each beside the
    library op of the same shape; bytes are the algorithmic minimum (every tensor read or written once per pass)."""
    import torch.nn.functional as F
    from autodist_b200.ops import functional as Fn
    rows = []
    N, C, Hh, W = 64, 256, 56, 56                                   # the ResNet stage-1 activation, 103 MB in bf16
    x = torch.randn(N, C, Hh, W, device=dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
    xh = x.permute(0, 2, 3, 1).contiguous()
    gamma, beta = torch.ones(C, device=dev), torch.zeros(C, device=dev)
    y = torch.empty_like(xh)
    mean, rstd = torch.empty(C, device=dev), torch.empty(C, device=dev)
    nbytes = xh.numel() * 2
    ms = _time(lambda: E.bn_fwd(xh, gamma, beta, None, y, mean, rstd, 1e-5, True, None, None, None, None, 0.1), flush=flush)
    ms_lib = _time(lambda: F.relu(F.batch_norm(x, None, None, gamma, beta, True, 0.1, 1e-5)), flush=flush)
    rows.append({"kernel": "bn_fwd+relu 64x56x56x256", "ms": round(ms, 4), "gbs": round(3 * nbytes / ms / 1e6, 1),
                 "library_ms": round(ms_lib, 4), "frac_of_measured_peak": round(3 * nbytes / ms / 1e6 / hbm, 3)})
    dy, dx = torch.randn_like(xh), torch.empty_like(xh)
    ms = _time(lambda: E.bn_bwd(dy, xh, y, mean, rstd, gamma, dx, None, True, None, None), flush=flush)
    rows.append({"kernel": "bn_bwd+relu 64x56x56x256", "ms": round(ms, 4), "gbs": round(7 * nbytes / ms / 1e6, 1),
                 "frac_of_measured_peak": round(7 * nbytes / ms / 1e6 / hbm, 3)})
    N, C, Hh, W = 64, 64, 112, 112                                   # the ResNet stem pool
    x = torch.randn(N, C, Hh, W, device=dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
    xh = x.permute(0, 2, 3, 1).contiguous()
    yo = torch.empty(N, 56, 56, C, dtype=torch.bfloat16, device=dev)
    nb = (xh.numel() + yo.numel()) * 2
    code = torch.empty(N, 56, 56, C, dtype=torch.uint8, device=dev)
    nb += code.numel()
    ms = _time(lambda: E.maxpool_fwd(xh, yo, code, 3, 2, 1), flush=flush)
    ms_lib = _time(lambda: F.max_pool2d(x, 3, 2, 1), flush=flush)
    rows.append({"kernel": "maxpool_fwd 3x3/2 64x112x112x64", "ms": round(ms, 4), "gbs": round(nb / ms / 1e6, 1),
                 "library_ms": round(ms_lib, 4), "frac_of_measured_peak": round(nb / ms / 1e6 / hbm, 3)})
    dyo, dxo = torch.randn_like(yo), torch.empty_like(xh)
    ms = _time(lambda: E.maxpool_bwd(code, dyo, dxo, 3, 2, 1), flush=flush)
    nb = (xh.numel() + yo.numel()) * 2 + code.numel()
    rows.append({"kernel": "maxpool_bwd 3x3/2 64x112x112x64", "ms": round(ms, 4), "gbs": round(nb / ms / 1e6, 1),
                 "frac_of_measured_peak": round(nb / ms / 1e6 / hbm, 3)})
    V, Hd, n = 793471, 512, 128 * 20 + 8192                          # LM1B tables and one step's lookups
    table = torch.randn(V, Hd, device=dev)
    ids = torch.randint(0, V, (n,), device=dev)
    out = torch.empty(n, Hd, dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: E.gather_rows_f32(table, ids, out), flush=flush)
    ms_lib = _time(lambda: F.embedding(ids, table).to(torch.bfloat16), flush=flush)
    rows.append({"kernel": f"gather_rows_f32 {n} rows x 512 of 793471", "ms": round(ms, 4), "gbs": round(n * Hd * 6 / ms / 1e6, 1),
                 "library_ms": round(ms_lib, 4), "frac_of_measured_peak": round(n * Hd * 6 / ms / 1e6 / hbm, 3)})
    acc = torch.zeros_like(table)
    uniq = torch.unique(ids)
    vals = torch.randn(uniq.numel(), Hd, device=dev)
    lr = torch.tensor([0.2], device=dev)
    ms = _time(lambda: Fn.sparse_rows_update_("adagrad", table, (uniq, vals), lr, acc), flush=flush)
    nb = uniq.numel() * Hd * 4 * 5
    rows.append({"kernel": f"sparse_rows_update adagrad {uniq.numel()} rows x 512", "ms": round(ms, 4), "gbs": round(nb / ms / 1e6, 1),
                 "frac_of_measured_peak": round(nb / ms / 1e6 / hbm, 3)})
    return rows


# (label, batch, Cin, H = W, Cout, k, stride, pad): the distinct convolutions of ResNet-101 at 224 x 224, batch 64
CONV_SHAPES = [("stem 7x7/2 3->64 @224", 64, 3, 224, 64, 7, 2, 3),
               ("s1 1x1 64->64 @56", 64, 64, 56, 64, 1, 1, 0), ("s1 3x3 64->64 @56", 64, 64, 56, 64, 3, 1, 1),
               ("s1 1x1 64->256 @56", 64, 64, 56, 256, 1, 1, 0), ("s1 1x1 256->64 @56", 64, 256, 56, 64, 1, 1, 0),
               ("s2 1x1 256->128 @56", 64, 256, 56, 128, 1, 1, 0), ("s2 3x3/2 128->128 @56", 64, 128, 56, 128, 3, 2, 1),
               ("s2 1x1/2 256->512 @56", 64, 256, 56, 512, 1, 2, 0), ("s2 3x3 128->128 @28", 64, 128, 28, 128, 3, 1, 1),
               ("s2 1x1 128->512 @28", 64, 128, 28, 512, 1, 1, 0), ("s2 1x1 512->128 @28", 64, 512, 28, 128, 1, 1, 0),
               ("s3 3x3/2 256->256 @28", 64, 256, 28, 256, 3, 2, 1), ("s3 3x3 256->256 @14", 64, 256, 14, 256, 3, 1, 1),
               ("s3 1x1 256->1024 @14", 64, 256, 14, 1024, 1, 1, 0), ("s3 1x1 1024->256 @14", 64, 1024, 14, 256, 1, 1, 0),
               ("s4 3x3/2 512->512 @14", 64, 512, 14, 512, 3, 2, 1), ("s4 3x3 512->512 @7", 64, 512, 7, 512, 3, 1, 1),
               ("s4 1x1 512->2048 @7", 64, 512, 7, 2048, 1, 1, 0), ("s4 1x1 2048->512 @7", 64, 2048, 7, 512, 1, 1, 0),
               ("vgg 3x3 64->64 @224 (batch 32)", 32, 64, 224, 64, 3, 1, 1), ("vgg 3x3 256->256 @56 (batch 32)", 32, 256, 56, 256, 3, 1, 1),
               ("vgg 3x3 512->512 @28 (batch 32)", 32, 512, 28, 512, 3, 1, 1)]


def _conv_rows(E, dev, flush, peaks, iters, only=""):
    """Forward, input gradient and weight gradient of the implicit-GEMM convolution at the ResNet-101 / VGG-16 layer shapes,
    beside the library convolution's forward pass (channels-last bf16). The roofline time of a layer is the slower of its
    FLOPs at the measured GEMM peak and its algorithmic bytes (each operand once) at the measured copy bandwidth."""
    import torch.nn.functional as F
    from autodist_b200.ops import functional as Fn
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    peak, hbm = peaks.get("bf16_tflops", 1656.4), peaks.get("hbm_gbs", 6518.6)
    rows = []
    for label, n, cin, hw, cout, k, stride, pad in CONV_SHAPES:
        if only and only not in label:
            continue
        oh = (hw + 2 * pad - k) // stride + 1
        w = (torch.randn(cout, k, k, cin, device=dev) / (cin * k * k) ** 0.5).to(torch.bfloat16)
        y = torch.empty(n, oh, oh, cout, dtype=torch.bfloat16, device=dev)
        dy = torch.randn(n, oh, oh, cout, device=dev).to(torch.bfloat16)
        flops = 2.0 * n * oh * oh * cout * cin * k * k
        row = {"kernel": f"conv {label}", "gflop": round(flops / 1e9, 1)}
        if cin % 8:
            img = torch.randn(n, cin, hw, hw, device=dev)
            _, _, hp, wp = Fn._rowtap_geometry(hw, hw, k, k, stride, pad)
            xp = torch.empty(n, hp, wp, 8, dtype=torch.bfloat16, device=dev)
            E.pad_image8(img, xp, pad)
            wr = F.pad(F.pad(w, (0, 8 - cin)).reshape(cout, k, k * 8), (0, 64 - k * 8)).contiguous()
            dwr = torch.empty(cout, k, 64, dtype=torch.float32, device=dev)
            ops_ = {"fprop": lambda: E.conv_rowtap_fprop(xp, wr, y, None, False, None, stride, err),
                    "wgrad": lambda: E.conv_rowtap_wgrad(dy, xp, dwr, stride, err)}
            xl = img.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            act_bytes = xp.numel() * 2
        else:
            x = torch.randn(n, hw, hw, cin, device=dev).to(torch.bfloat16)
            dx = torch.empty_like(x)
            dw = torch.empty(cout, k, k, cin, dtype=torch.float32, device=dev)
            ops_ = {"fprop": lambda: E.conv_fprop(x, w, y, None, False, None, stride, pad, err),
                    "dgrad": lambda: E.conv_dgrad(dy, w, dx, stride, pad, err),
                    "wgrad": lambda: E.conv_wgrad(dy, x, dw, stride, pad, err, False)}
            xl = x.permute(0, 3, 1, 2)
            act_bytes = x.numel() * 2
        nbytes = act_bytes + y.numel() * 2 + w.numel() * 2
        roof_ms = max(flops / (peak * 1e9), nbytes / (hbm * 1e6))
        for name, fn in ops_.items():
            ms = _time(fn, iters=iters, flush=flush)
            row[name + "_us"] = round(ms * 1e3, 1)
            row[name + "_tflops"] = round(flops / ms / 1e9, 1)
            row[name + "_frac_of_roofline"] = round(roof_ms / ms, 3)
        wl = w.permute(0, 3, 1, 2)
        ms = _time(lambda: F.conv2d(xl, wl, None, stride, pad), iters=iters, flush=flush)
        row["library_fprop_us"] = round(ms * 1e3, 1)
        row["roofline_us"] = round(roof_ms * 1e3, 1)
        rows.append(row)
    assert err.item() == 0, f"a convolution kernel gave up waiting (code {err.item()})"
    return rows


def _layer_rows(E, dev, iters, trace):
    """The twelve GEMMs of one BERT-large encoder layer (4096 tokens, hidden 1024, FFN 4096) with the epilogues the model
    uses, each launched ``iters`` times back to back with warm caches (no L2 flush: the training step runs them that way);
    the kernel is the one the binding picks (``bn = 0``). ``trace``: also print the phase marks of the two-CTA kernel for the
    FFN1 product (nanoseconds per CTA, median / maximum over the CTAs)."""
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    T, H, F = 4096, 1024, 4096
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    x, wqkv, wo, w1, w2 = bf(T, H), bf(3 * H, H), bf(H, H), bf(F, H), bf(H, F)
    qkv, att, o = torch.empty(T, 3 * H, dtype=torch.bfloat16, device=dev), bf(T, H), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    u = torch.empty(T, F, dtype=torch.bfloat16, device=dev)
    g, y = torch.empty_like(u), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    bq, bo, b1, b2 = (torch.randn(n, device=dev) for n in (3 * H, H, F, H))
    dy, dg, dx = bf(T, H), torch.empty(T, F, dtype=torch.bfloat16, device=dev), torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    gw1, gw2, gwo, gwq = (torch.zeros(*s, device=dev) for s in ((F, H), (H, F), (H, H), (3 * H, H)))
    datt, dqkv = torch.empty(T, H, dtype=torch.bfloat16, device=dev), bf(T, 3 * H)

    def G(a, b, c, a_mn=False, b_mn=False, epi=0, bias=None, c2=None, aux=None, beta=0.0):
        E.gemm(a, b, c, a_mn, b_mn, epi, bias, c2, aux, 1.0, beta, err, 0)

    products = [("QKV forward (bias)", lambda: G(x, wqkv, qkv, epi=1, bias=bq)),
                ("attention output forward (bias)", lambda: G(att, wo, o, epi=1, bias=bo)),
                ("FFN1 forward (bias + GELU, two outputs)", lambda: G(x, w1, u, epi=2, bias=b1, c2=g)),
                ("FFN2 forward (bias)", lambda: G(g, w2, y, epi=1, bias=b2)),
                ("FFN2 dX (x GELU')", lambda: G(dy, w2, dg, b_mn=True, epi=3, aux=u)),
                ("FFN2 dW (fp32 +=)", lambda: G(dy, g, gw2, a_mn=True, b_mn=True, beta=1.0)),
                ("FFN1 dX", lambda: G(dg, w1, dx, b_mn=True)),
                ("FFN1 dW (fp32 +=)", lambda: G(dg, x, gw1, a_mn=True, b_mn=True, beta=1.0)),
                ("attention output dX", lambda: G(dy, wo, datt, b_mn=True)),
                ("attention output dW (fp32 +=)", lambda: G(dy, att, gwo, a_mn=True, b_mn=True, beta=1.0)),
                ("QKV dX (+ residual gradient)", lambda: G(dqkv, wqkv, dx, b_mn=True, epi=4, aux=dx)),
                ("QKV dW (fp32 +=)", lambda: G(dqkv, x, gwq, a_mn=True, b_mn=True, beta=1.0))]

    def hot(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters * 1e3

    rows, total = [], 0.0
    for name, fn in products:
        us = hot(fn)
        total += us
        rows.append({"product": name, "us": round(us, 1)})
    rows.append({"product": "sum of the twelve", "us": round(total, 1),
                 "pair_kernel": os.environ.get("AUTODIST_GEMM_PAIR", "1") != "0", "tma_store": os.environ.get("AUTODIST_GEMM_TMA_STORE", "1") != "0"})
    lib = [("cuBLAS addmm QKV forward", lambda: torch.addmm(bq.to(torch.bfloat16), x, wqkv.t(), out=qkv)),
           ("cuBLAS addmm FFN1 forward (bias only)", lambda: torch.addmm(b1.to(torch.bfloat16), x, w1.t(), out=u)),
           ("cuBLAS addmm FFN2 forward", lambda: torch.addmm(b2.to(torch.bfloat16), g, w2.t(), out=y))]
    for name, fn in lib:
        rows.append({"product": name, "us": round(hot(fn), 1)})
    if trace:
        import statistics
        a, b, c = bf(T, H), bf(F, H), torch.empty(T, F, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            E.gemm(a, b, c, False, False, 0, None, None, None, 1.0, 0.0, err, 512)
        marks = torch.zeros(torch.cuda.get_device_properties(0).multi_processor_count, 8, dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        E.gemm_set_trace(marks)
        E.gemm(a, b, c, False, False, 0, None, None, None, 1.0, 0.0, err, 512)
        torch.cuda.synchronize()
        E.gemm_set_trace(None)
        t = marks.cpu()
        t = t[t[:, 0] > 0]
        t0 = int(t[:, 0].min())
        lead = t[0::2]
        med = lambda xs: int(statistics.median(xs))
        rows.append({"trace": "two-CTA kernel 4096x4096x1024, ns", "ctas": int(t.shape[0]),
                     "set_up_done_median": med([int(v) - t0 for v in lead[:, 1]]),
                     "first_stage_full_median": med([int(v) - t0 for v in lead[:, 2]]),
                     "last_mma_committed_median_max": [med([int(v) - t0 for v in lead[:, 3]]), max(int(v) - t0 for v in lead[:, 3])],
                     "mma_thread_waited_for_stages_median": med(lead[:, 4].tolist()),
                     "mma_thread_waited_for_accumulator_median": med(lead[:, 5].tolist()),
                     "first_epilogue_warp_busy_median": med(t[:, 6].tolist())})
    assert err.item() == 0, f"a GEMM kernel gave up waiting (code {err.item()})"
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--only", default="", help="run only the GEMM shapes whose label contains this text")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--group", default="all", choices=["all", "gemm", "bert", "cnn", "conv", "layer"],
                    help="gemm: GEMM shapes; bert: LayerNorm / Adam; cnn: batch-norm, max-pool, row gather, sparse-row update; "
                         "conv: implicit-GEMM convolution at the ResNet-101 / VGG-16 layer shapes; layer: the twelve GEMMs of one "
                         "BERT-large encoder layer with their epilogues, warm caches")
    ap.add_argument("--trace", action="store_true", help="with --group layer: phase marks of the two-CTA kernel")
    args = ap.parse_args()
    from autodist_b200 import ops
    E = ops.ext(required=True)
    dev = "cuda"
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peaks = {}
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
    rows = []
    T = 4096
    shapes = [("qkv fwd", T, 3072, 1024, False, False), ("ffn1 fwd", T, 4096, 1024, False, False),
              ("ffn2 fwd", T, 1024, 4096, False, False), ("out fwd", T, 1024, 1024, False, False),
              ("ffn1 dX", T, 1024, 4096, False, True), ("ffn2 dX", T, 4096, 1024, False, True),
              ("ffn1 dW", 4096, 1024, T, True, True), ("ffn2 dW", 1024, 4096, T, True, True),
              ("square 8192", 8192, 8192, 8192, False, False)]
    if args.small:
        shapes = shapes[:2]
    if args.only:
        shapes = [s for s in shapes if args.only in s[0]]
    if args.group == "layer":
        for r in _layer_rows(E, dev, max(args.iters, 5), args.trace):
            print(json.dumps(r))
        return
    if args.group == "conv":
        rows = _conv_rows(E, dev, flush, peaks, args.iters, args.only)
        for r in rows:
            print(json.dumps(r))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f, indent=1)
        return
    if args.group in ("bert", "cnn"):
        shapes = []
    for name, M, N, K, a_mn, b_mn in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device=dev).to(torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device=dev).to(torch.bfloat16)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        for bn in (512, 256, 128):          # 512: the 256 x 256 tile of the two-CTA kernel
            if bn == 512 and (M < 256 or N < 256):
                continue
            ms = _time(lambda: E.gemm(a, b, c, a_mn, b_mn, 0, None, None, None, 1.0, 0.0, err, bn), iters=args.iters, flush=flush)
            A = a.t() if a_mn else a
            B = b if b_mn else b.t()
            ms_lib = _time(lambda: torch.matmul(A, B, out=c), iters=args.iters, flush=flush)
            fl = 2.0 * M * N * K
            rows.append({"kernel": f"gemm {name} {M}x{N}x{K} bn{bn}", "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                         "cublas_ms": round(ms_lib, 4), "cublas_tflops": round(fl / ms_lib / 1e9, 1),
                         "frac_of_measured_peak": round(fl / ms / 1e9 / peaks.get("bf16_tflops", 1656.4), 3)})
    if args.only:
        for r in rows:
            print(json.dumps(r))
        return
    hbm = peaks.get("hbm_gbs", 6518.6)
    if args.group in ("all", "cnn"):
        rows += _cnn_rows(E, dev, flush, hbm)
    if args.group in ("gemm", "cnn"):
        for r in rows:
            print(json.dumps(r))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f, indent=1)
        return
    # bandwidth-bound kernels
    H = 1024
    x = torch.randn(T * 8, H, device=dev).to(torch.bfloat16)
    res = torch.randn_like(x.float()).to(torch.bfloat16)
    g, bta = torch.ones(H, device=dev), torch.zeros(H, device=dev)
    z, y = torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(T * 8, device=dev), torch.empty(T * 8, device=dev)
    ms = _time(lambda: E.ln_fwd(x, res, g, bta, z, y, mean, rstd, 1e-12, 0.1, 1, None), flush=flush)
    rows.append({"kernel": "ln_fwd 32768x1024 (+res+dropout)", "ms": round(ms, 4), "gbs": round(4 * x.numel() * 2 / ms / 1e6, 1),
                 "frac_of_measured_peak": round(4 * x.numel() * 2 / ms / 1e6 / peaks.get("hbm_gbs", 6518.6), 3)})
    part = torch.zeros(E.ln_bwd_part_floats(H), device=dev)
    dg, db = torch.empty(H, device=dev), torch.empty(H, device=dev)
    ms = _time(lambda: E.ln_bwd(y, z, mean, rstd, g, None, x, res, part, dg, db, 0.1, 1, None, False, None), flush=flush)
    rows.append({"kernel": "ln_bwd 32768x1024 (+dropout)", "ms": round(ms, 4), "gbs": round(4 * x.numel() * 2 / ms / 1e6, 1),
                 "frac_of_measured_peak": round(4 * x.numel() * 2 / ms / 1e6 / peaks.get("hbm_gbs", 6518.6), 3)})
    n = 128 << 20
    p, gr, m, v = (torch.zeros(n, device=dev) for _ in range(4))
    p16 = torch.empty(n, dtype=torch.bfloat16, device=dev)
    lr = torch.tensor([1e-3], device=dev)
    st = torch.ones(1, dtype=torch.int64, device=dev)
    ms = _time(lambda: E.adam_update(p, gr, m, v, p16, lr, 0.9, 0.999, 1e-8, 0.0, False, st, 1.0))
    rows.append({"kernel": "adam 128M params", "ms": round(ms, 4), "gbs": round(n * 30 / ms / 1e6, 1),
                 "frac_of_measured_peak": round(n * 30 / ms / 1e6 / peaks.get("hbm_gbs", 6518.6), 3)})
    for r in rows:
        print(json.dumps(r))
    assert err.item() == 0
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
