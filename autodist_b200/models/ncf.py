"""NeuMF recommendation model (reference: ``examples/benchmark/utils/recommendation/neumf_model.py:200-251``).

One user table and one item table of width ``mf_dim + layers[0] // 2``; the first ``mf_dim`` columns feed the
generalised matrix-factorisation branch (element-wise product), the rest feed the MLP branch (concatenated, then
``layers[1:]`` with ReLU). The two branches are concatenated into one logit. Embedding gradients are row-sparse so a
PS / Parallax strategy moves only the looked-up rows; ``dense_gradient=True`` gives dense gradients for all-reduce
strategies (reference: ``examples/benchmark/ncf.py:325-326``).
"""
from dataclasses import dataclass, field
from typing import List

import torch
from torch import nn
import torch.nn.functional as F

from autodist_b200.ops.functional import Linear


@dataclass
class NeuMFConfig:
    num_users: int = 138493                 # ml-20m
    num_items: int = 26744
    mf_dim: int = 64
    layers: List[int] = field(default_factory=lambda: [256, 256, 128, 64])
    dense_gradient: bool = False

    @classmethod
    def tiny(cls, **kw):
        d = dict(num_users=200, num_items=120, mf_dim=8, layers=[64, 32, 16, 8])
        d.update(kw)
        return cls(**d)


class NeuMF(nn.Module):
    _autodist_leaf = True

    def __init__(self, config: NeuMFConfig = NeuMFConfig()):
        super().__init__()
        c = self.config = config
        if c.layers[0] % 2:
            raise ValueError("layers[0] is split between the user and the item embedding and must be even")
        width = c.mf_dim + c.layers[0] // 2
        self.user_emb = nn.Parameter(torch.randn(c.num_users, width) * 0.01)
        self.item_emb = nn.Parameter(torch.randn(c.num_items, width) * 0.01)
        self.mlp = nn.ModuleList(Linear(a, b) for a, b in zip(c.layers[:-1], c.layers[1:]))
        self.head = nn.Linear(c.mf_dim + c.layers[-1], 1)

    def sparse_grad_parameters(self):
        return [] if self.config.dense_gradient else [self.user_emb, self.item_emb]

    def logits(self, users, items):
        c = self.config
        sparse = not c.dense_gradient
        u = F.embedding(users, self.user_emb, sparse=sparse)
        i = F.embedding(items, self.item_emb, sparse=sparse)
        gmf = u[:, :c.mf_dim] * i[:, :c.mf_dim]
        x = torch.cat([u[:, c.mf_dim:], i[:, c.mf_dim:]], 1)
        for layer in self.mlp:
            x = F.relu(layer(x)).to(gmf.dtype)
        return self.head(torch.cat([gmf, x], 1)).squeeze(1)

    def forward(self, users, items, labels, weights=None):
        """Binary cross-entropy on (user, item) pairs; ``weights`` masks padded duplicates as the reference's
        ``valid_point_mask`` does."""
        loss = F.binary_cross_entropy_with_logits(self.logits(users, items), labels.float(), reduction="none")
        if weights is None:
            return loss.mean()
        w = weights.float()
        return (loss * w).sum() / w.sum().clamp_min(1.0)


def synthetic_interactions(batch, config, num_neg=4, seed=0):
    """One positive per ``num_neg`` uniformly sampled negatives, ids uniform over the tables (synthetic ml-20m shape)."""
    g = torch.Generator().manual_seed(seed)
    users = torch.randint(0, config.num_users, (batch,), generator=g)
    items = torch.randint(0, config.num_items, (batch,), generator=g)
    labels = (torch.arange(batch) % (num_neg + 1) == 0).float()
    return {"users": users, "items": items, "labels": labels}


def hit_rate_and_ndcg(scores, top_k=10):
    """Leave-one-out ranking metrics: ``scores[:, 0]`` is the held-out positive, the other columns sampled negatives."""
    rank = (scores[:, 1:] >= scores[:, :1]).sum(1)                            # items ranked ahead of the positive
    hit = rank < top_k
    ndcg = torch.where(hit, 1.0 / torch.log2(rank.float() + 2.0), torch.zeros_like(rank, dtype=torch.float32))
    return hit.float().mean().item(), ndcg.mean().item()
