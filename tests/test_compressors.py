"""Compressor math against plain restatements (single replica backend: the collective is the identity)."""
import torch

from autodist_b200.kernel.synchronization.compressor import Compressor, orthogonalize_
from autodist_b200.parallel.comm import LocalBackend


class Bucket:
    def __init__(self, shapes):
        self._shapes = shapes

    def member_shapes(self):
        return self._shapes


def test_factory():
    for name in ("NoneCompressor", "HorovodCompressor", "HorovodCompressorEF", "PowerSGDCompressor"):
        assert type(Compressor.create(name, Bucket([(4,)]))).__name__ == name


def test_horovod_ef_residual_persists():
    torch.manual_seed(0)
    c = Compressor.create("HorovodCompressorEF", Bucket([(1000,)]))
    be = LocalBackend()
    g = torch.randn(1000) * 1e-3
    total_sent = torch.zeros(1000)
    for _ in range(50):
        total_sent += c.reduce(g.clone(), be)
    # with error feedback the accumulated transmitted signal tracks the accumulated true signal
    assert (total_sent - 50 * g).abs().max() < 2e-6
    plain = Compressor.create("HorovodCompressor", Bucket([(1000,)]))
    out = plain.reduce(g.clone(), be)
    assert torch.equal(out, g.half().float())


def test_orthogonalize():
    p = torch.randn(50, 4)
    orthogonalize_(p)
    assert torch.allclose(p.t() @ p, torch.eye(4), atol=1e-5)


def test_power_sgd_rank1_exact_on_rank1_matrix():
    torch.manual_seed(1)
    u, v = torch.randn(32, 1), torch.randn(1, 24)
    M = u @ v
    bias = torch.randn(24)
    c = Compressor.create("PowerSGDCompressor", Bucket([(32, 24), (24,)]), rank=1)
    flat = torch.cat([M.reshape(-1), bias])
    out = c.reduce(flat.clone(), LocalBackend())
    assert torch.allclose(out[:32 * 24].view(32, 24), M, atol=1e-4)
    assert torch.equal(out[32 * 24:], bias)
    assert c.error.abs().max() < 1e-4


def test_power_sgd_error_feedback_converges():
    torch.manual_seed(2)
    M = torch.randn(16, 12)
    c = Compressor.create("PowerSGDCompressor", Bucket([(16, 12)]), rank=2)
    sent = torch.zeros(16, 12)
    for _ in range(200):
        sent += c.reduce(M.reshape(-1).clone(), LocalBackend()).view(16, 12)
    assert (sent / 200 - M).norm() / M.norm() < 0.1
