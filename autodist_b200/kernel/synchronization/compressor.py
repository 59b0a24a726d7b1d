"""Gradient compressors applied around a bucket's all-reduce.

Capability parity with ``autodist/kernel/synchronization/compressor.py:30-284``
plus the behaviour the reference left unfinished:

* ``HorovodCompressor`` really narrows the wire format (fp16 by default, bf16 on
  request) - the reference casts to float32, a no-op for fp32 gradients
  (``compressor.py:191-198``);
* the error-feedback residual is a buffer that persists across steps - in the
  reference it is a Python attribute rebuilt with the graph (``compressor.py:120-143``);
* ``PowerSGDCompressor`` is enabled (commented out at ``compressor.py:208-284``)
  in its published form: warm-started ``Q``, ``P = M Q``, mean all-reduce of
  ``P``, orthogonalisation, ``Q = M^T P``, mean all-reduce of ``Q``, result
  ``P Q^T`` and residual ``M - P Q^T``.

A compressor works on one bucket (the flat concatenation of a group's
gradients). It talks to the communication backend through
``compressed_all_reduce_mean_`` so that a backend with fused kernels can do the
cast and the residual update inside the collective.
"""
import os
from abc import ABC, abstractmethod

import torch

_WIRE = {"fp16": torch.float16, "float16": torch.float16, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}


def wire_dtype():
    return _WIRE[os.environ.get("AUTODIST_COMPRESS_DTYPE", "fp16").lower()]


class Compressor(ABC):
    """``reduce(flat, backend)`` returns the mean of ``flat`` over all replicas (in place)."""

    def __init__(self, bucket):
        self.bucket = bucket

    @abstractmethod
    def reduce(self, flat, backend):
        raise NotImplementedError

    def state_dict(self):
        return {}

    def load_state_dict(self, state):
        return

    @classmethod
    def create(cls, name, *args, **kwargs):
        stack = list(cls.__subclasses__())
        while stack:
            sub = stack.pop()
            if sub.__name__ == name:
                return sub(*args, **kwargs)
            stack.extend(sub.__subclasses__())
        raise ValueError(f"{name} is not a valid compressor name")


class NoneCompressor(Compressor):
    def reduce(self, flat, backend):
        return backend.compressed_all_reduce_mean_(flat, None, None)


class HorovodCompressor(Compressor):
    """Narrow floating-point gradients to 16 bits on the wire, widen the mean back."""

    def reduce(self, flat, backend):
        wd = wire_dtype() if flat.dtype in (torch.float32, torch.float64) else None
        return backend.compressed_all_reduce_mean_(flat, wd, None)


class CompressorEF(Compressor):
    """Error feedback: what the compression lost this step is added to the next step's gradient."""

    def __init__(self, bucket):
        super().__init__(bucket)
        self.error = None

    def _residual(self, flat):
        if self.error is None or self.error.shape != flat.shape or self.error.device != flat.device:
            self.error = torch.zeros_like(flat)
        return self.error

    def state_dict(self):
        return {"error": self.error}

    def load_state_dict(self, state):
        self.error = state.get("error")


class HorovodCompressorEF(CompressorEF, HorovodCompressor):
    def reduce(self, flat, backend):
        if flat.dtype not in (torch.float32, torch.float64):
            return backend.compressed_all_reduce_mean_(flat, None, None)
        return backend.compressed_all_reduce_mean_(flat, wire_dtype(), self._residual(flat))


def orthogonalize_(p, eps=1e-8):
    """Modified Gram-Schmidt on the columns of ``p`` (in place)."""
    for i in range(p.shape[1]):
        col = p[:, i:i + 1]
        col /= col.norm() + eps
        if i + 1 < p.shape[1]:
            rest = p[:, i + 1:]
            rest -= col @ (col.t() @ rest)
    return p


class PowerSGDCompressor(CompressorEF):
    """Rank-``r`` low-rank all-reduce (Vogels et al., 2019) with error feedback.

    Matrices (every bucket member with at least two dimensions, reshaped to
    ``[d0, -1]``) travel as ``P`` then ``Q`` factors; vectors travel uncompressed
    in the same flat message as the ``P`` factors.
    """

    def __init__(self, bucket, rank=1, seed=1905_13727):
        super().__init__(bucket)
        self.rank = max(1, int(rank))
        self.seed = seed
        self.q = {}
        self._layout = None

    def _plan(self, flat):
        """Bucket members as (offset, numel, matrix shape or None)."""
        if self._layout is None:
            out, off = [], 0
            for shape in self.bucket.member_shapes():
                numel = 1
                for d in shape:
                    numel *= d
                mat = (shape[0], numel // shape[0]) if len(shape) >= 2 and min(shape[0], numel // shape[0]) > self.rank \
                    else None
                out.append((off, numel, mat))
                off += numel
            self._layout = out
        return self._layout

    def _q_for(self, idx, n, like):
        if idx not in self.q:
            g = torch.Generator(device="cpu").manual_seed(self.seed + idx)
            self.q[idx] = torch.randn(n, self.rank, generator=g, dtype=torch.float32).to(like.device, like.dtype)
        return self.q[idx]

    def reduce(self, flat, backend):
        layout = self._plan(flat)
        err = self._residual(flat)
        if flat.is_cuda and flat.dtype == torch.float32 and self.rank <= 4:
            return self._reduce_cuda(flat, err, layout, backend)
        flat.add_(err)
        mats = [(i, off, numel, mat) for i, (off, numel, mat) in enumerate(layout) if mat is not None]
        vecs = [(off, numel) for off, numel, mat in layout if mat is None]
        # message 1: all P factors followed by all uncompressed members
        p_sizes = [mat[0] * self.rank for _, _, _, mat in mats]
        msg1 = flat.new_empty(sum(p_sizes) + sum(n for _, n in vecs))
        cursor, p_views = 0, []
        for (i, off, numel, (m, n)), psz in zip(mats, p_sizes):
            M = flat[off:off + numel].view(m, n)
            pv = msg1[cursor:cursor + psz].view(m, self.rank)
            torch.matmul(M, self._q_for(i, n, flat), out=pv)
            p_views.append(pv)
            cursor += psz
        for off, numel in vecs:
            msg1[cursor:cursor + numel].copy_(flat[off:off + numel])
            cursor += numel
        backend.compressed_all_reduce_mean_(msg1, None, None)
        # message 2: all Q factors
        q_sizes = [mat[1] * self.rank for _, _, _, mat in mats]
        msg2 = flat.new_empty(sum(q_sizes))
        cursor, q_views = 0, []
        for (i, off, numel, (m, n)), pv, qsz in zip(mats, p_views, q_sizes):
            orthogonalize_(pv)
            M = flat[off:off + numel].view(m, n)
            qv = msg2[cursor:cursor + qsz].view(n, self.rank)
            torch.matmul(M.t(), pv, out=qv)
            q_views.append(qv)
            cursor += qsz
        if mats:
            backend.compressed_all_reduce_mean_(msg2, None, None)
        # decompress, update residual, write the result over the bucket
        err.zero_()
        for (i, off, numel, (m, n)), pv, qv in zip(mats, p_views, q_views):
            M = flat[off:off + numel].view(m, n)
            approx = pv @ qv.t()
            err[off:off + numel].view(m, n).copy_(M - approx)
            M.copy_(approx)
            self.q[i] = qv.clone()
        cursor = sum(p_sizes)
        for off, numel in vecs:
            flat[off:off + numel].copy_(msg1[cursor:cursor + numel])
            cursor += numel
        return flat

    def _reduce_cuda(self, flat, err, layout, backend):
        """Same algorithm on the hand-written kernels: three bandwidth-bound passes per matrix (P, Q, decompress)."""
        from autodist_b200 import ops
        E = ops.ext(required=True)
        mats = [(i, off, numel, mat) for i, (off, numel, mat) in enumerate(layout) if mat is not None]
        vecs = [(off, numel) for off, numel, mat in layout if mat is None]
        r = self.rank
        p_sizes = [mat[0] * r for _, _, _, mat in mats]
        msg1 = flat.new_empty(sum(p_sizes) + sum(n for _, n in vecs))
        cursor, p_views = 0, []
        for (i, off, numel, (m, n)), psz in zip(mats, p_sizes):
            M = flat[off:off + numel].view(m, n)
            pv = msg1[cursor:cursor + psz].view(m, r)
            E.psgd_p(M, err[off:off + numel].view(m, n), self._q_for(i, n, flat).contiguous(), pv)
            p_views.append(pv)
            cursor += psz
        for off, numel in vecs:
            flat[off:off + numel].add_(err[off:off + numel])
            msg1[cursor:cursor + numel].copy_(flat[off:off + numel])
            cursor += numel
        backend.compressed_all_reduce_mean_(msg1, None, None)
        q_sizes = [mat[1] * r for _, _, _, mat in mats]
        msg2 = flat.new_empty(max(sum(q_sizes), 1))
        cursor, q_views = 0, []
        for (i, off, numel, (m, n)), pv, qsz in zip(mats, p_views, q_sizes):
            orthogonalize_(pv)
            qv = msg2[cursor:cursor + qsz].view(n, r)
            E.psgd_q(flat[off:off + numel].view(m, n), pv, qv)
            q_views.append(qv)
            cursor += qsz
        if mats:
            backend.compressed_all_reduce_mean_(msg2[:sum(q_sizes)], None, None)
        for off, numel in vecs:
            err[off:off + numel].zero_()
        for (i, off, numel, (m, n)), pv, qv in zip(mats, p_views, q_views):
            E.psgd_d(flat[off:off + numel].view(m, n), err[off:off + numel].view(m, n), pv.contiguous(), qv.contiguous())
            self.q[i] = qv.clone()
        cursor = sum(p_sizes)
        for off, numel in vecs:
            flat[off:off + numel].copy_(msg1[cursor:cursor + numel])
            cursor += numel
        return flat

    def state_dict(self):
        return {"error": self.error, "q": self.q}

    def load_state_dict(self, state):
        self.error = state.get("error")
        self.q = state.get("q", {})
