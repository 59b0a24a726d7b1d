"""Small models of the reference's getting-started examples (``examples/linear_regression.py``,
``image_classifier.py``, ``sentiment_classifier.py``) and the NCF recommender (``examples/benchmark/ncf.py``)."""
import torch
from torch import nn
import torch.nn.functional as F


class FashionCNN(nn.Module):
    """Conv32 - MaxPool - Flatten - Dropout - Dense10 (``examples/image_classifier.py``)."""

    def __init__(self, num_classes=10):
        super().__init__()
        self.conv = nn.Conv2d(1, 32, 3)
        self.drop = nn.Dropout(0.5)
        self.fc = nn.Linear(32 * 13 * 13, num_classes)

    def logits(self, images):
        h = F.max_pool2d(F.relu(self.conv(images)), 2).flatten(1)
        return self.fc(self.drop(h))

    def forward(self, images, labels=None):
        """Loss when ``labels`` are given (session-style programs), logits otherwise (``training.Model``)."""
        out = self.logits(images)
        return out if labels is None else F.cross_entropy(out, labels)


class SentimentClassifier(nn.Module):
    """Embedding 10000x16 -> mean pool -> 16 -> 16 -> 1 (``examples/sentiment_classifier.py:12-112``)."""

    def __init__(self, vocab=10000, dim=16, sparse=True):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim, sparse=sparse)
        self.fc1 = nn.Linear(dim, 16)
        self.fc2 = nn.Linear(16, 1)

    def forward(self, ids, labels):
        h = self.emb(ids).mean(1)
        logit = self.fc2(F.relu(self.fc1(h))).squeeze(-1)
        return F.binary_cross_entropy_with_logits(logit, labels)


def NeuMF(num_users, num_items, mf_dim=64, layers=(256, 256, 128, 64), sparse=True):
    """Neural matrix factorisation with positional arguments; the model itself lives in ``models.ncf``."""
    from autodist_b200.models.ncf import NeuMF as _NeuMF, NeuMFConfig
    return _NeuMF(NeuMFConfig(num_users, num_items, mf_dim, list(layers), dense_gradient=not sparse))


class NeuMF(nn.Module):
    """Neural matrix factorisation (``examples/benchmark/utils/recommendation/neumf_model.py:200-251``): user / item
    embeddings of width ``mf_dim + layers[0] / 2`` sliced into a GMF part and an MLP part, MLP tower, one logit."""

    def __init__(self, num_users, num_items, mf_dim=64, layers=(256, 256, 128, 64), sparse=True):
        super().__init__()
        self.mf_dim = mf_dim
        width = mf_dim + layers[0] // 2
        self.user = nn.Embedding(num_users, width, sparse=sparse)
        self.item = nn.Embedding(num_items, width, sparse=sparse)
        self.mlp = nn.ModuleList([nn.Linear(layers[i], layers[i + 1]) for i in range(len(layers) - 1)])
        self.out = nn.Linear(mf_dim + layers[-1], 1)

    def forward(self, users, items, labels):
        u, i = self.user(users), self.item(items)
        gmf = u[:, :self.mf_dim] * i[:, :self.mf_dim]
        h = torch.cat([u[:, self.mf_dim:], i[:, self.mf_dim:]], 1)
        for layer in self.mlp:
            h = F.relu(layer(h))
        logit = self.out(torch.cat([gmf, h], 1)).squeeze(-1)
        return F.binary_cross_entropy_with_logits(logit, labels)
