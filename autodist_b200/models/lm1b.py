"""LM1B-shape language model (reference: ``examples/lm1b/language_model.py:17-148``).

Embedding ``[V, 512]`` -> dropout -> one LSTM layer (2048 units, 512-wide projection, forget bias +1) unrolled over
``num_steps`` -> sampled softmax over ``num_sampled`` log-uniform negatives. The embedding and softmax tables are the
large row-sparse variables a PartitionedPS strategy shards; LSTM gradients are clipped by global norm (10) through
``minimize(..., clip_global_norm=...)`` and the loss is scaled by ``num_steps`` as in the reference.
"""
import math
from dataclasses import dataclass

import torch
from torch import nn
import torch.nn.functional as F

from autodist_b200.ops.functional import linear, lstm_cell, sparse_lookup


@dataclass
class LM1BConfig:
    vocab_size: int = 793471
    emb_size: int = 512
    state_size: int = 2048
    projected_size: int = 512
    num_sampled: int = 8192
    num_steps: int = 20
    keep_prob: float = 0.9
    max_grad_norm: float = 10.0

    @classmethod
    def tiny(cls):
        return cls(vocab_size=2000, emb_size=64, state_size=128, projected_size=64, num_sampled=64, num_steps=8)


def log_uniform_sample(num_sampled, vocab, generator=None, device="cpu"):
    """Log-uniform (Zipfian) candidate sampler: ``P(k) = log((k+2)/(k+1)) / log(V+1)``; returns ids and P(ids)."""
    u = torch.rand(num_sampled, generator=generator, device=device)
    ids = (torch.exp(u * math.log(vocab + 1.0)) - 1.0).long().clamp_(0, vocab - 1)
    return ids


def log_uniform_prob(ids, vocab):
    idf = ids.float()
    return torch.log((idf + 2.0) / (idf + 1.0)) / math.log(vocab + 1.0)


class LM1B(nn.Module):
    _autodist_leaf = True

    def __init__(self, config: LM1BConfig = LM1BConfig()):
        super().__init__()
        c = self.config = config
        self.emb = nn.Parameter(torch.empty(c.vocab_size, c.emb_size).uniform_(-0.05, 0.05))
        self.softmax_w = nn.Parameter(torch.empty(c.vocab_size, c.projected_size).uniform_(-0.05, 0.05))
        self.softmax_b = nn.Parameter(torch.zeros(c.vocab_size))
        self.W = nn.Parameter(torch.empty(4 * c.state_size, c.emb_size + c.projected_size).uniform_(-0.05, 0.05))
        self.B = nn.Parameter(torch.zeros(4 * c.state_size))
        self.W_P = nn.Parameter(torch.empty(c.projected_size, c.state_size).uniform_(-0.05, 0.05))
        self._gen = None

    def sparse_grad_parameters(self):
        return [self.emb, self.softmax_w, self.softmax_b]

    def sparse_lookup_parameters(self):
        """Tables read only through ``sparse_lookup``: an engine may keep them as row shards instead of replicas."""
        return [self.emb, self.softmax_w]

    def dense_parameters(self):
        return [self.W, self.B, self.W_P]

    def forward(self, x, y):
        """``x``, ``y``: int64 ``[batch, num_steps]`` token ids and next-token targets. Returns the scaled loss."""
        c = self.config
        Bsz, T = x.shape
        dt = torch.bfloat16 if x.is_cuda else torch.float32
        inputs = sparse_lookup(self.emb, x).to(dt)               # row-sparse gradient: only the looked-up rows travel
        if self.training and c.keep_prob < 1.0:
            inputs = F.dropout(inputs, 1.0 - c.keep_prob)
        h = torch.zeros(Bsz, c.projected_size, dtype=dt, device=x.device)
        cell = torch.zeros(Bsz, c.state_size, dtype=torch.float32, device=x.device)
        outs = []
        for t in range(T):
            gates = linear(torch.cat([inputs[:, t], h], 1), self.W, self.B)
            cell, hidden = lstm_cell(gates, cell, 1.0)
            h = linear(hidden.to(dt), self.W_P)
            outs.append(h)
        out = torch.stack(outs, 1).reshape(Bsz * T, c.projected_size)
        if self.training and c.keep_prob < 1.0:
            out = F.dropout(out, 1.0 - c.keep_prob)
        # sampled softmax: true class + shared log-uniform negatives, logits corrected by -log(expected count)
        targets = y.reshape(-1)
        if x.is_cuda:
            gen = None            # the device's default generator: its state survives capture into a CUDA graph
        else:
            if self._gen is None:
                self._gen = torch.Generator()
                self._gen.manual_seed(1234)
            gen = self._gen
        neg = log_uniform_sample(c.num_sampled, c.vocab_size, gen, x.device)
        true_w = sparse_lookup(self.softmax_w, targets).to(dt)
        true_logit = (out * true_w).sum(1).float() + self.softmax_b[targets] - torch.log(
            c.num_sampled * log_uniform_prob(targets, c.vocab_size))
        neg_w = sparse_lookup(self.softmax_w, neg).to(dt)
        neg_logit = linear(out, neg_w).float() + self.softmax_b[neg]        # [B*T, 512] x [8192, 512]^T on the tcgen05 GEMM
        neg_logit = neg_logit - torch.log(c.num_sampled * log_uniform_prob(neg, c.vocab_size))
        neg_logit = neg_logit.masked_fill(neg[None, :] == targets[:, None], -1e9)     # remove accidental hits
        logits = torch.cat([true_logit[:, None], neg_logit], 1)
        loss = F.cross_entropy(logits, torch.zeros_like(targets))
        return loss * c.num_steps


def zipf_tokens(batch, num_steps, vocab, s=1.1, seed=0):
    """Token ids drawn from a Zipf(s) distribution over the vocabulary (synthetic LM1B input)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(batch, num_steps + 1, generator=g, dtype=torch.float64)
    # inverse-CDF of the continuous approximation of Zipf(s) on [1, V]
    a = 1.0 - s
    ids = ((u * (vocab ** a - 1.0) + 1.0) ** (1.0 / a)).long().clamp_(1, vocab) - 1
    return {"x": ids[:, :-1].contiguous(), "y": ids[:, 1:].contiguous()}
