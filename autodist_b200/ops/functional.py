"""Autograd-visible wrappers of the hand-written kernels for models that keep using ``torch.autograd``.

``linear`` runs forward, dX and dW on the tcgen05 GEMM (bf16 operands, fp32 accumulation; the weight gradient is
produced in fp32). On CPU tensors the same functions fall back to the plain PyTorch expression, which is also the
numerics reference of the tests.
"""
import warnings

import torch
import torch.nn.functional as F

from autodist_b200 import ops

_err = {}


def _error_flag(device):
    if device not in _err:
        _err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err[device]


def check_errors():
    for dev, flag in _err.items():
        code = int(flag.item())
        if code:
            raise RuntimeError(f"a GEMM kernel on {dev} gave up waiting (code {code})")


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, activation):
        E = ops.ext(required=True)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        w16 = _bf16_weight(weight)
        y = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        err = _error_flag(x.device)
        pre = None
        b32 = bias.float().contiguous() if bias is not None else None
        gathered = getattr(weight, "_gathered", None) if activation is None else None
        ctx.gathered = gathered
        if gathered is not None:
            # the weight's row shards stay with their owners: B tiles are fetched over NVLink inside the GEMM
            E.gemm_gathered_b(x2, gathered["ptrs"], gathered["rows"], y, 1 if b32 is not None else 0, b32, err, 0)
        elif activation == "gelu":
            pre = torch.empty_like(y)
            E.gemm(x2, w16, pre, False, False, 2, b32 if b32 is not None else torch.zeros(weight.shape[0], device=x.device),
                   y, None, 1.0, 0.0, err, 0)
        elif b32 is not None:
            E.gemm(x2, w16, y, False, False, 1, b32, None, None, 1.0, 0.0, err, 0)
        else:
            E.gemm(x2, w16, y, False, False, 0, None, None, None, 1.0, 0.0, err, 0)
        ctx.save_for_backward(x2, w16, pre)
        ctx.weight = weight
        _count_use(ctx, weight, 1)
        ctx.has_bias = bias is not None
        ctx.shape = shape
        ctx.w_dtype = weight.dtype
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        E = ops.ext(required=True)
        x2, w16, pre = ctx.saved_tensors
        err = _error_flag(dy.device)
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        if pre is not None:
            du = torch.empty_like(dy2)
            E.gelu_bwd(dy2, pre, du)
            dy2 = du
        dx = torch.empty_like(x2)
        if ctx.gathered is not None:
            E.gemm_gathered_bt(dy2, ctx.gathered["ptrs"], ctx.gathered["rows"], w16.shape[1], dx, err)   # dX = dY . W, W from its owners
        else:
            E.gemm(dy2, w16, dx, False, True, 0, None, None, None, 1.0, 0.0, err, 0)      # dX = dY . W
        acc = _direct_grad(ctx.weight)
        if acc is not None:
            E.gemm(dy2, x2, acc, True, True, 0, None, None, None, 1.0, 1.0, err, 0)       # dW += dY^T . X, in the gradient buffer
            dw = None
        else:
            dw = torch.empty(w16.shape, dtype=torch.float32, device=dy.device)
            E.gemm(dy2, x2, dw, True, True, 0, None, None, None, 1.0, 0.0, err, 0)        # dW = dY^T . X
        db = None
        if ctx.has_bias:
            n = dy2.shape[1]
            if n % 8 == 0:
                db = torch.empty(n, dtype=torch.float32, device=dy.device)
                part = torch.empty(E.colsum_parts(dy2.shape[0]) * n, dtype=torch.float32, device=dy.device)
                E.keyed_colsum(dy2, None, part, db, 1, False)
            else:
                db = dy2.float().sum(0)
        if dw is None:
            _grad_written(ctx.weight)
        return dx.view(ctx.shape).to(dy.dtype), None if dw is None else dw.to(ctx.w_dtype), db, None


def linear(x, weight, bias=None, activation=None):
    """``activation(x @ weight.T + bias)`` with ``activation`` in ``{None, "gelu"}`` (tanh form)."""
    if x.is_cuda and x.shape[-1] % 8 == 0 and (weight.shape[0] % 8 == 0):
        return _LinearFn.apply(x, weight, bias, activation)
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    return F.gelu(y, approximate="tanh") if activation == "gelu" else y


class Linear(torch.nn.Linear):
    """Drop-in ``nn.Linear`` whose CUDA path is the tcgen05 GEMM."""

    def forward(self, x):
        return linear(x, self.weight, self.bias)


class _LSTMCellFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, c_prev, forget_bias):
        E = ops.ext(required=True)
        gates = gates.float().contiguous()
        c_prev = c_prev.float().contiguous()
        c = torch.empty_like(c_prev)
        h = torch.empty(c_prev.shape, dtype=torch.bfloat16, device=c_prev.device)
        E.lstm_cell_fwd(gates, c_prev, c, h, forget_bias)
        ctx.save_for_backward(gates, c_prev, c)
        ctx.fb = forget_bias
        return c, h

    @staticmethod
    def backward(ctx, dc_next, dh):
        E = ops.ext(required=True)
        gates, c_prev, c = ctx.saved_tensors
        dh = torch.zeros_like(c) if dh is None else dh.float().contiguous()
        dgates = torch.empty_like(gates)
        dc_prev = torch.empty_like(c)
        E.lstm_cell_bwd(gates, c_prev, c, dh, None if dc_next is None else dc_next.float().contiguous(), dgates, dc_prev, ctx.fb)
        return dgates, dc_prev, None


def lstm_cell(gates, c_prev, forget_bias=1.0):
    """Pointwise part of an LSTM step: ``gates`` [B, 4S] in the order i, j, f, o -> ``(c_new fp32, h bf16)``."""
    if gates.is_cuda:
        return _LSTMCellFn.apply(gates, c_prev, forget_bias)
    i, j, f, o = gates.float().chunk(4, 1)
    c = torch.sigmoid(f + forget_bias) * c_prev + torch.sigmoid(i) * torch.tanh(j)
    return c, torch.sigmoid(o) * torch.tanh(c)


def clip_by_global_norm_(grads, max_norm, weights=None, all_reduce=None):
    """Scale fp32 CUDA gradients in place so that their joint L2 norm is at most ``max_norm``; the norm stays on the
    device. ``weights`` weighs each tensor's squared sum (replicated tensors count once across ranks);
    ``all_reduce`` (optional callable) sums the squared norm over ranks."""
    E = ops.ext(required=True)
    acc = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
    for k, g in enumerate(grads):
        E.sumsq(g, acc, 1.0 if weights is None else weights[k])
    if all_reduce is not None:
        all_reduce(acc)
    for g in grads:
        E.clip_scale(g, acc, max_norm)
    return acc


def _nhwc(x):
    """bf16 ``[N, H, W, C]`` contiguous view / copy of a logical ``[N, C, H, W]`` tensor (free for channels-last bf16)."""
    return x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()


def _bf16_weight(weight):
    """bf16 copy of a parameter: the engine's flat compute copy when the parameter lives in flat buffers, else a cast."""
    view = getattr(weight, "_bf16_view", None)
    if view is not None and view.device == weight.device:
        return view
    return weight.detach().to(torch.bfloat16).contiguous()


def _direct_grad(param):
    """The fp32 gradient buffer of ``param`` when its owner (a flat-buffer engine) asked for gradients to be accumulated
    in place by the producing kernel instead of travelling through autograd's accumulation; else ``None``."""
    if not getattr(param, "_direct_grad", False):
        return None                 # (asked first: reading .grad of a non-leaf tensor makes PyTorch warn)
    g = param.grad
    if g is not None and g.dtype == torch.float32 and g.is_contiguous() and g.is_cuda:
        return g
    return None


def _count_use(ctx, param, index):
    """Forward side of the direct accumulation: remember that one more kernel call will add into ``param``'s gradient."""
    if ctx.needs_input_grad[index] and getattr(param, "_direct_grad", False):
        param._pending_uses = getattr(param, "_pending_uses", 0) + 1


def _grad_written(param):
    """Backward side: one pending call has added its part; after the last one tell the owner that the gradient is final."""
    param._pending_uses = getattr(param, "_pending_uses", 1) - 1
    hook = getattr(param, "_grad_ready_hook", None)
    if hook is not None and param._pending_uses <= 0:
        hook(param)


def _colsum(E, dy2):
    n = dy2.shape[1]
    db = torch.empty(n, dtype=torch.float32, device=dy2.device)
    part = torch.empty(E.colsum_parts(dy2.shape[0]) * n, dtype=torch.float32, device=dy2.device)
    E.keyed_colsum(dy2, None, part, db, 1, False)
    return db


def _rowtap_geometry(h, w, kh, kw, stride, padding):
    """Padded-image extents of the first-layer path: the halo is written out and rows are long enough for the last
    64-element read of every output column."""
    oh, ow = (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1
    hp = max(h + 2 * padding, (oh - 1) * stride + kh)
    wp = max(w + 2 * padding, (ow - 1) * stride + 8)
    return oh, ow, hp, wp + (wp & 1)


class GradFork:
    """Meeting point of the two consumers of a forked tensor (the input of a residual block feeds the block's first
    convolution and its skip connection). Whichever consumer's backward runs first leaves its gradient here and returns
    none; the second adds it inside its own kernel (the input-gradient convolution's epilogue) and returns the sum, so
    the fork costs no elementwise pass of its own."""
    __slots__ = ("grad",)

    def __init__(self):
        self.grad = None

    def take(self):
        g, self.grad = self.grad, None
        return g


class _ForkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, box):
        ctx.box = box
        ctx.set_materialize_grads(False)
        return x.view_as(x), x.view_as(x)

    @staticmethod
    def backward(ctx, ga, gb):
        # a gradient left behind (its partner never ran, or could not fuse the add) still counts
        parts = [g for g in (ga, gb, ctx.box.take()) if g is not None]
        if not parts:
            return None, None
        out = parts[0]
        for g in parts[1:]:
            out = out + g
        return out, None


def fork(x):
    """Two aliases of ``x`` for its two consumers plus the ``GradFork`` both pass to their kernels (``conv2d(fork=...)``,
    ``batch_norm(fork=...)``); ``(x, x, None)`` where no gradient flows."""
    if not (x.is_cuda and x.requires_grad and torch.is_grad_enabled()):
        return x, x, None
    box = GradFork()
    a, b = _ForkFn.apply(x, box)
    return a, b, box


class _ConvFn(torch.autograd.Function):
    """2-D convolution as an implicit GEMM on tcgen05 (``csrc/conv_tcgen05.cu``): forward, input gradient and weight
    gradient read the channels-last bf16 activations in place through TMA boxes, one per filter tap; bias, ReLU and the
    per-channel sums a following batch-norm needs are fused into the forward epilogue. ``weight`` is ``[Cout, KH, KW, Cin]``."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, relu, stats, fork=None):
        E = ops.ext(required=True)
        ctx.fork = fork
        cout, kh, kw, cin = weight.shape
        err = _error_flag(x.device)
        b32 = bias.detach().float().contiguous() if bias is not None else None
        w16 = _bf16_weight(weight)
        ctx.rowtap = cin % 8 != 0
        if ctx.rowtap:
            n, _, h, w = x.shape
            oh, ow, hp, wp = _rowtap_geometry(h, w, kh, kw, stride, padding)
            xh = torch.empty(n, hp, wp, 8, dtype=torch.bfloat16, device=x.device)
            E.pad_image8(x, xh, padding)
            wr = F.pad(F.pad(w16, (0, 8 - cin)).reshape(cout, kh, kw * 8), (0, 64 - kw * 8)).contiguous()
            y = torch.empty(n, oh, ow, cout, dtype=torch.bfloat16, device=x.device)
            E.conv_rowtap_fprop(xh, wr, y, b32, relu, stats, stride, err)
        else:
            xh = _nhwc(x)
            n, h, w, _ = xh.shape
            oh, ow = (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1
            y = torch.empty(n, oh, ow, cout, dtype=torch.bfloat16, device=x.device)
            E.conv_fprop(xh, w16, y, b32, relu, stats, stride, padding, err)
        ctx.save_for_backward(xh, w16, y if relu else None)
        ctx.weight, ctx.bias = weight, bias
        _count_use(ctx, weight, 1)
        if bias is not None:
            _count_use(ctx, bias, 2)
        ctx.geom = (stride, padding, tuple(weight.shape), tuple(x.shape))
        ctx.has_bias = bias is not None
        ctx.dtypes = (x.dtype, weight.dtype)
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        E = ops.ext(required=True)
        xh, w16, y = ctx.saved_tensors
        stride, padding, (cout, kh, kw, cin), x_shape = ctx.geom
        err = _error_flag(dy.device)
        dyh = _nhwc(dy)
        db = None
        bias = ctx.bias
        acc_b = _direct_grad(bias) if bias is not None else None
        if bias is not None:
            # bias gradient (and the ReLU mask) in one pass over dy
            db = acc_b if acc_b is not None else torch.empty(cout, dtype=torch.float32, device=dy.device)
            masked = torch.empty_like(dyh) if y is not None else None
            E.relu_bwd_colsum(dyh, y, masked, db, acc_b is not None)
            dyh = masked if masked is not None else dyh
        elif y is not None:
            masked = torch.empty_like(dyh)
            E.relu_bwd(dyh, y, masked)
            dyh = masked
        dx = None
        if ctx.rowtap:
            dwr = torch.empty(cout, kh, 64, dtype=torch.float32, device=dy.device)
            E.conv_rowtap_wgrad(dyh, xh, dwr, stride, err)
            dw = dwr[:, :, :kw * 8].reshape(cout, kh, kw, 8)[..., :cin].contiguous()
            if ctx.needs_input_grad[0]:
                w_oihw = w16.float().permute(0, 3, 1, 2)
                dx = torch.nn.grad.conv2d_input(x_shape, w_oihw, dy.float(), stride, padding).to(ctx.dtypes[0])
        else:
            acc = _direct_grad(ctx.weight)
            if acc is not None:
                E.conv_wgrad(dyh, xh, acc, stride, padding, err, True)       # split-K atomics land in the parameter's gradient buffer
                dw = None
            else:
                dw = torch.empty(cout, kh, kw, cin, dtype=torch.float32, device=dy.device)
                E.conv_wgrad(dyh, xh, dw, stride, padding, err, False)
            if ctx.needs_input_grad[0]:
                dxh = torch.empty_like(xh)
                other = ctx.fork.take() if ctx.fork is not None else None
                E.conv_dgrad(dyh, w16, dxh, stride, padding, err, None if other is None else _nhwc(other))
                dx = dxh.permute(0, 3, 1, 2).to(ctx.dtypes[0])
                if ctx.fork is not None and other is None:
                    ctx.fork.grad, dx = dx, None            # first of the two consumers: the other one adds this in its kernel
        if dw is None:
            _grad_written(ctx.weight)
        if acc_b is not None:
            _grad_written(bias)
            db = None
        return dx, None if dw is None else dw.to(ctx.dtypes[1]), db, None, None, None, None, None


def conv2d(x, weight, bias=None, stride=1, padding=0, relu=False, stats=None, fork=None):
    """Convolution of a logical ``[N, C, H, W]`` tensor with a ``[Cout, KH, KW, Cin]`` weight (+ bias, + ReLU).

    On a GPU it runs on the implicit-GEMM kernels when the channel counts allow it: ``Cin`` and ``Cout`` multiples of 8,
    or ``Cin <= 8`` with ``KW <= 8`` (the first layer of an image network, whose input is padded to 8 channels). ``stats``
    (fp32 ``[2, Cout]``, zeroed by the caller) receives the per-channel sum and sum of squares of the output. Other shapes
    and CPU tensors use the library convolution."""
    cout, kh, kw, cin = weight.shape
    own = x.is_cuda and cout % 8 == 0 and stride in (1, 2) and kh * kw <= 49 and (cin % 8 == 0 or (cin <= 8 and kw <= 8))
    if own:
        return _ConvFn.apply(x, weight, bias, int(stride), int(padding), bool(relu), stats, fork)
    y = F.conv2d(x, weight.permute(0, 3, 1, 2).to(x.dtype), None if bias is None else bias.to(x.dtype), stride, padding)
    y = F.relu(y) if relu else y
    if stats is not None:
        with torch.no_grad():
            yf = y.float()
            stats[0] += yf.sum((0, 2, 3))
            stats[1] += (yf * yf).sum((0, 2, 3))
    return y


class _BatchNormFn(torch.autograd.Function):
    """Training-mode batch-norm over channels-last activations on the hand-written kernels, with the tail of a residual
    block fused in: ``y = relu?(bn(x) + residual)``. ``sums`` (fp32 ``[2, C]``: sum and sum of squares per channel, as the
    convolution's epilogue leaves them) skips the statistics pass."""

    @staticmethod
    def forward(ctx, x, gamma, beta, residual, eps, relu, sums, running, fork=None):
        E = ops.ext(required=True)
        ctx.fork = fork
        run_mean, run_var, batches, momentum = running if running is not None else (None, None, None, 0.0)
        xh = _nhwc(x)                                                            # [N, H, W, C]
        c = xh.shape[-1]
        y = torch.empty_like(xh)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        g32, b32 = gamma.detach().float().contiguous(), beta.detach().float().contiguous()
        res = _nhwc(residual) if residual is not None else None
        E.bn_fwd(xh, g32, b32, res, y, mean, rstd, eps, relu, sums, run_mean, run_var, batches, momentum)
        ctx.save_for_backward(xh, y, mean, rstd, g32)
        ctx.params = (gamma, beta)
        ctx.set_materialize_grads(False)                     # mean / rstd carry no gradient: no zero tensors for them
        _count_use(ctx, gamma, 1)
        _count_use(ctx, beta, 2)
        ctx.relu = relu
        ctx.has_res = residual is not None
        ctx.dtypes = (x.dtype, gamma.dtype, residual.dtype if residual is not None else None)
        ctx.mark_non_differentiable(mean, rstd)
        return y.permute(0, 3, 1, 2), mean, rstd

    @staticmethod
    def backward(ctx, dy, _dm, _dr):
        E = ops.ext(required=True)
        xh, y, mean, rstd, g32 = ctx.saved_tensors
        if dy is None:
            return (None,) * 9
        dyh = _nhwc(dy)
        dx = torch.empty_like(xh)
        dres = None
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = torch.empty_like(xh) if ctx.relu else dyh                    # without a ReLU the residual gradient is dy itself
        gamma, beta = ctx.params
        acc_g, acc_b = _direct_grad(gamma), _direct_grad(beta)
        direct = acc_g is not None and acc_b is not None
        sums = E.bn_bwd(dyh, xh, y, mean, rstd, g32, dx, dres if ctx.relu else None, ctx.relu, acc_g if direct else None,
                        acc_b if direct else None)
        dr = dres.permute(0, 3, 1, 2).to(ctx.dtypes[2]) if dres is not None else None
        if ctx.fork is not None and dr is not None:
            other = ctx.fork.take()
            if other is None:
                ctx.fork.grad, dr = dr, None            # the residual's other consumer adds this in its input-gradient kernel
            else:
                dr = dr + other
        if direct:
            _grad_written(gamma)
            _grad_written(beta)
            return dx.permute(0, 3, 1, 2).to(ctx.dtypes[0]), None, None, dr, None, None, None, None, None
        return dx.permute(0, 3, 1, 2).to(ctx.dtypes[0]), sums[1].to(ctx.dtypes[1]), sums[0].to(ctx.dtypes[1]), dr, None, None, None, None, None


def batch_norm(x, gamma, beta, running_mean=None, running_var=None, training=True, momentum=0.1, eps=1e-5, relu=False,
               residual=None, sums=None, num_batches_tracked=None, fork=None):
    """``relu?(batch_norm(x) + residual)`` of an NCHW / channels-last tensor; updates the running statistics like
    ``F.batch_norm``. ``sums``: per-channel sum / sum of squares of ``x`` when a preceding kernel already produced them."""
    if not (x.is_cuda and training and x.shape[1] % 8 == 0):
        y = F.batch_norm(x, running_mean, running_var, gamma.to(x.dtype) if x.dtype != gamma.dtype and not x.is_cuda else gamma,
                         beta, training, momentum, eps)
        if residual is not None:
            y = y + residual
        return F.relu(y) if relu else y
    running = None
    if running_mean is not None and running_mean.dtype == torch.float32 and running_var.dtype == torch.float32:
        running = (running_mean, running_var, num_batches_tracked, float(momentum))     # folded into the statistics kernel
    y, mean, rstd = _BatchNormFn.apply(x, gamma, beta, residual, eps, relu, sums, running, fork)
    if running is None and running_mean is not None:
        with torch.no_grad():
            n = x.numel() // x.shape[1]
            var = (1.0 / (rstd * rstd) - eps).clamp_(min=0) * (n / max(n - 1, 1))
            running_mean.mul_(1 - momentum).add_(mean.to(running_mean.dtype), alpha=momentum)
            running_var.mul_(1 - momentum).add_(var.to(running_var.dtype), alpha=momentum)
        if num_batches_tracked is not None:
            num_batches_tracked.add_(1)
    return y


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, stride, pad):
        E = ops.ext(required=True)
        xh = x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        n, h, w, c = xh.shape
        ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = torch.empty(n, ho, wo, c, dtype=torch.bfloat16, device=x.device)
        code = torch.empty(n, ho, wo, c, dtype=torch.uint8, device=x.device)
        E.maxpool_fwd(xh, y, code, k, stride, pad)
        ctx.save_for_backward(code)
        ctx.geom = (k, stride, pad)
        ctx.x_shape = tuple(xh.shape)
        ctx.x_dtype = x.dtype
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        E = ops.ext(required=True)
        (code,) = ctx.saved_tensors
        dx = torch.empty(ctx.x_shape, dtype=torch.bfloat16, device=dy.device)
        E.maxpool_bwd(code, dy.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous(), dx, *ctx.geom)
        return dx.permute(0, 3, 1, 2).to(ctx.x_dtype), None, None, None


def max_pool2d(x, kernel_size, stride=None, padding=0):
    stride = stride or kernel_size
    if x.is_cuda and x.shape[1] % 8 == 0:
        return _MaxPoolFn.apply(x, int(kernel_size), int(stride), int(padding))
    return F.max_pool2d(x, kernel_size, stride, padding)


class _SparseLookupFn(torch.autograd.Function):
    """Rows ``ids`` of an fp32 table as bf16 (gather with the cast fused); the gradient is row-sparse like
    ``F.embedding(sparse=True)`` so only the looked-up rows travel to the table's owner."""

    @staticmethod
    def forward(ctx, table, ids):
        E = ops.ext(required=True)
        flat = ids.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
        E.gather_rows_f32(table.detach(), flat, out)
        ctx.save_for_backward(flat)
        ctx.shape = tuple(table.shape)
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        vals = dy.reshape(flat.numel(), -1).float()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                                   # the library's notice that invariants are unchecked
            return torch.sparse_coo_tensor(flat[None], vals, ctx.shape, check_invariants=False), None


class _ShardedLookupFn(torch.autograd.Function):
    """Lookup in a table that is kept as one row shard per rank (``parallel.fused_engine.ShardedRows``): rows are gathered
    from their owners inside the kernel; the backward pass adds the gradient rows straight into the owners' shards, so the
    table has no gradient tensor at all. ``anchor`` is a dummy that requires grad, so that autograd runs the backward pass."""

    @staticmethod
    def forward(ctx, anchor, handle, ids):
        ctx.handle = handle
        ctx.save_for_backward(ids)
        return handle.lookup(ids).view(*ids.shape, handle.H)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        ctx.handle.push(ids, dy.reshape(-1, ctx.handle.H))
        return None, None, None


_ANCHORS = {}


def sparse_lookup(table, ids):
    """``F.embedding(ids, table, sparse=True)`` returning bf16 on CUDA (fp32 elsewhere).

    A module that reads a table only through this function may list it in ``sparse_lookup_parameters()``; an engine can
    then keep the table as one row shard per rank and attach the shard handle to the parameter (``_sparse_rows``), in which
    case the lookup and its gradient run on the peer-memory kernels."""
    handle = getattr(table, "_sparse_rows", None)
    if handle is not None and ids.is_cuda:
        anchor = _ANCHORS.get(ids.device)
        if anchor is None:
            anchor = _ANCHORS[ids.device] = torch.zeros((), device=ids.device, requires_grad=True)
        return _ShardedLookupFn.apply(anchor, handle, ids)
    if table.is_cuda and table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] % 8 == 0:
        return _SparseLookupFn.apply(table, ids)
    return F.embedding(ids, table, sparse=True)


_SPARSE_KINDS = {"sgd": 0, "lazy_adam": 1, "adagrad": 2}


def sparse_rows_update_(kind, table, grad, lr, state1=None, state2=None, step=None, betas=(0.9, 0.999), eps=1e-8,
                        grad_scale=1.0, table_bf16=None):
    """Apply a row-sparse gradient to ``table`` in place, touching only the rows that carry a gradient.

    ``kind``: ``"sgd"``, ``"lazy_adam"`` (moments of untouched rows do not decay; ``step`` is the int64 device counter
    already incremented for this step) or ``"adagrad"``. ``grad`` is a sparse COO tensor (it is coalesced first: the
    kernel needs unique rows) or a ``(rows, values)`` pair that is already unique. ``lr`` is a float or a device
    tensor. The reference reaches the same updates through TensorFlow's ``ResourceSparseApply*`` family
    (``autodist/kernel/common/op_info.py:24-117``)."""
    E = ops.ext(required=True)
    if isinstance(grad, tuple):
        rows, vals = grad
    else:
        g = grad.coalesce()
        rows, vals = g.indices()[0], g.values()
    if not torch.is_tensor(lr):
        lr = torch.tensor([float(lr)], dtype=torch.float32, device=table.device)
    E.sparse_rows_update(table, state1, state2, table_bf16, rows.contiguous(), vals.float().contiguous(), _SPARSE_KINDS[kind], lr,
                         betas[0], betas[1], eps, step, grad_scale)
    return table
