"""Autograd-visible wrappers of the hand-written kernels for models that keep using ``torch.autograd``.

``linear`` runs forward, dX and dW on the tcgen05 GEMM (bf16 operands, fp32 accumulation; the weight gradient is
produced in fp32). On CPU tensors the same functions fall back to the plain PyTorch expression, which is also the
numerics reference of the tests.
"""
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


def _aligned(x, weight):
    return x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 or (x.shape[-1] % 8 == 0 and weight.shape[0] >= 1)


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
