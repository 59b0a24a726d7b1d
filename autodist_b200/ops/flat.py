"""Flat parameter storage for models that run on the hand-written kernels.

All parameters of a model live in one fp32 master buffer, one bf16 compute copy
and one fp32 gradient buffer; every variable starts on a 16-byte boundary of all
three, so that a range of variables is a valid bucket for the all-reduce kernel
and ``.grad`` of a parameter is a view the backward GEMMs write straight into.
"""
import torch


def _round_up(n, m):
    return (n + m - 1) // m * m


class FlatParams:
    def __init__(self, named_params, device, grad_alloc=None, align=8, master_alloc=None, p16_alloc=None):
        self.names, self.params, self.offsets, self.numels = [], [], {}, {}
        off = 0
        for name, p in named_params:
            self.names.append(name)
            self.params.append(p)
            self.offsets[name] = off
            self.numels[name] = p.numel()
            off = _round_up(off + p.numel(), align)
        self.total = _round_up(off, 64)
        self.device = torch.device(device)
        self.master = master_alloc(self.total) if master_alloc is not None else \
            torch.zeros(self.total, dtype=torch.float32, device=device)
        self.p16 = p16_alloc(self.total) if p16_alloc is not None else \
            torch.zeros(self.total, dtype=torch.bfloat16, device=device)
        self.grad = grad_alloc(self.total) if grad_alloc is not None else \
            torch.zeros(self.total, dtype=torch.float32, device=device)
        self.w32, self.w16, self.g = {}, {}, {}
        with torch.no_grad():
            for name, p in zip(self.names, self.params):
                o, n = self.offsets[name], p.numel()
                view = self.master[o:o + n].view(p.shape)
                view.copy_(p.data.to(device=device, dtype=torch.float32))
                p.data = view
                self.w32[name] = view
                self.w16[name] = self.p16[o:o + n].view(p.shape)
                self.g[name] = self.grad[o:o + n].view(p.shape)
                p.grad = self.g[name]
        self.refresh_bf16()

    def refresh_bf16(self):
        if self.device.type == "cuda":
            from autodist_b200 import ops
            ops.ext(required=True).cast_f32_bf16(self.master, self.p16)
        else:
            self.p16.copy_(self.master)

    def range_of(self, names):
        """[lo, hi) of the flat buffers covered by consecutive variables ``names`` (hi is padded to alignment)."""
        lo = self.offsets[names[0]]
        last = names[-1]
        idx = self.names.index(last)
        hi = self.offsets[self.names[idx + 1]] if idx + 1 < len(self.names) else self.total
        return lo, hi

    def rebind_grad(self, new_grad):
        """Move the gradient views onto another buffer (e.g. symmetric memory) of the same length."""
        assert new_grad.numel() >= self.total
        self.grad = new_grad
        for name, p in zip(self.names, self.params):
            o, n = self.offsets[name], p.numel()
            self.g[name] = self.grad[o:o + n].view(p.shape)
            p.grad = self.g[name]
