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
        w16 = weight.to(torch.bfloat16).contiguous()
        y = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        err = _error_flag(x.device)
        pre = None
        b32 = bias.float().contiguous() if bias is not None else None
        if activation == "gelu":
            pre = torch.empty_like(y)
            E.gemm(x2, w16, pre, False, False, 2, b32 if b32 is not None else torch.zeros(weight.shape[0], device=x.device),
                   y, None, 1.0, 0.0, err, 0)
        elif b32 is not None:
            E.gemm(x2, w16, y, False, False, 1, b32, None, None, 1.0, 0.0, err, 0)
        else:
            E.gemm(x2, w16, y, False, False, 0, None, None, None, 1.0, 0.0, err, 0)
        ctx.save_for_backward(x2, w16, pre)
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
        E.gemm(dy2, w16, dx, False, True, 0, None, None, None, 1.0, 0.0, err, 0)          # dX = dY . W
        dw = torch.empty(w16.shape, dtype=torch.float32, device=dy.device)
        E.gemm(dy2, x2, dw, True, True, 0, None, None, None, 1.0, 0.0, err, 0)            # dW = dY^T . X
        db = None
        if ctx.has_bias:
            n = dy2.shape[1]
            if n % 8 == 0:
                db = torch.empty(n, dtype=torch.float32, device=dy.device)
                part = torch.empty(E.colsum_parts(dy2.shape[0]) * n, dtype=torch.float32, device=dy.device)
                E.keyed_colsum(dy2, None, part, db, 1, False)
            else:
                db = dy2.float().sum(0)
        return dx.view(ctx.shape).to(dy.dtype), dw.to(ctx.w_dtype), db, None


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


class _ConvGemmFn(torch.autograd.Function):
    """2-D convolution as im2col + tcgen05 GEMM (forward, input gradient, weight gradient), channels-last bf16."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding):
        E = ops.ext(required=True)
        cout, cin, kh, kw = weight.shape
        xh = x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()            # [N, H, W, C]
        n, h, w, _ = xh.shape
        ho, wo = (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1
        w2 = weight.permute(0, 2, 3, 1).reshape(cout, kh * kw * cin).to(torch.bfloat16).contiguous()
        cols = torch.empty(n * ho * wo, kh * kw * cin, dtype=torch.bfloat16, device=x.device)
        E.im2col(xh, cols, kh, kw, stride, padding)
        y = torch.empty(n * ho * wo, cout, dtype=torch.bfloat16, device=x.device)
        err = _error_flag(x.device)
        if bias is not None:
            E.gemm(cols, w2, y, False, False, 1, bias.float().contiguous(), None, None, 1.0, 0.0, err, 0)
        else:
            E.gemm(cols, w2, y, False, False, 0, None, None, None, 1.0, 0.0, err, 0)
        ctx.save_for_backward(xh, w2)
        ctx.geom = (kh, kw, stride, padding, ho, wo, cin, cout)
        ctx.has_bias = bias is not None
        ctx.w_dtype, ctx.x_dtype = weight.dtype, x.dtype
        return y.view(n, ho, wo, cout).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        E = ops.ext(required=True)
        xh, w2 = ctx.saved_tensors
        kh, kw, stride, padding, ho, wo, cin, cout = ctx.geom
        n = xh.shape[0]
        err = _error_flag(dy.device)
        dy2 = dy.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous().view(n * ho * wo, cout)
        cols = torch.empty(n * ho * wo, kh * kw * cin, dtype=torch.bfloat16, device=dy.device)
        E.im2col(xh, cols, kh, kw, stride, padding)                            # recomputed: cheaper than keeping it
        dw2 = torch.empty(cout, kh * kw * cin, dtype=torch.float32, device=dy.device)
        E.gemm(dy2, cols, dw2, True, True, 0, None, None, None, 1.0, 0.0, err, 0)      # dW = dY^T . cols
        dcols = cols                                                            # reuse the buffer
        E.gemm(dy2, w2, dcols, False, True, 0, None, None, None, 1.0, 0.0, err, 0)     # dcols = dY . W
        dx = torch.empty_like(xh)
        E.col2im(dcols, dx, kh, kw, stride, padding)
        dw = dw2.view(cout, kh, kw, cin).permute(0, 3, 1, 2).to(ctx.w_dtype)
        db = dy2.float().sum(0) if ctx.has_bias else None
        return dx.permute(0, 3, 1, 2).to(ctx.x_dtype), dw, db, None, None


def conv2d(x, weight, bias=None, stride=1, padding=0):
    """Convolution on the hand-written kernels when the channel counts allow it (multiples of 8), else the library."""
    cout, cin = weight.shape[0], weight.shape[1]
    if x.is_cuda and cin % 8 == 0 and cout % 8 == 0:
        return _ConvGemmFn.apply(x, weight, bias, int(stride), int(padding))
    return F.conv2d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), stride, padding)


class _BatchNormFn(torch.autograd.Function):
    """Training-mode batch-norm (+ optional ReLU) over channels-last activations on the hand-written kernels."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, relu):
        E = ops.ext(required=True)
        xh = x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()            # [N, H, W, C]
        c = xh.shape[-1]
        y = torch.empty_like(xh)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        g32, b32 = gamma.float().contiguous(), beta.float().contiguous()
        E.bn_fwd(xh, g32, b32, y, mean, rstd, eps, relu)
        ctx.save_for_backward(xh, y, mean, rstd, g32)
        ctx.relu = relu
        ctx.dtypes = (x.dtype, gamma.dtype)
        ctx.mark_non_differentiable(mean, rstd)
        return y.permute(0, 3, 1, 2), mean, rstd

    @staticmethod
    def backward(ctx, dy, _dm, _dr):
        E = ops.ext(required=True)
        xh, y, mean, rstd, g32 = ctx.saved_tensors
        dyh = dy.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        dx = torch.empty_like(xh)
        sums = E.bn_bwd(dyh, xh, y, mean, rstd, g32, dx, ctx.relu)
        return dx.permute(0, 3, 1, 2).to(ctx.dtypes[0]), sums[1].to(ctx.dtypes[1]), sums[0].to(ctx.dtypes[1]), None, None


def batch_norm(x, gamma, beta, running_mean=None, running_var=None, training=True, momentum=0.1, eps=1e-5, relu=False):
    """Batch-norm (+ ReLU) of an NCHW / channels-last tensor; updates the running statistics like ``F.batch_norm``."""
    if not (x.is_cuda and training and x.shape[1] % 8 == 0):
        y = F.batch_norm(x, running_mean, running_var, gamma.to(x.dtype) if x.dtype != gamma.dtype and not x.is_cuda else gamma,
                         beta, training, momentum, eps)
        return F.relu(y) if relu else y
    y, mean, rstd = _BatchNormFn.apply(x, gamma, beta, eps, relu)
    if running_mean is not None:
        with torch.no_grad():
            n = x.numel() // x.shape[1]
            var = (1.0 / (rstd * rstd) - eps).clamp_(min=0) * (n / max(n - 1, 1))
            running_mean.mul_(1 - momentum).add_(mean.to(running_mean.dtype), alpha=momentum)
            running_var.mul_(1 - momentum).add_(var.to(running_var.dtype), alpha=momentum)
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


def sparse_lookup(table, ids):
    """``F.embedding(ids, table, sparse=True)`` returning bf16 on CUDA (fp32 elsewhere)."""
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
