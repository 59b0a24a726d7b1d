"""Model cases of the strategy x case matrix (mirrors the spirit of the reference's
``tests/integration/cases/c0.py`` ... ``c7.py``): each case builds a single-device program,
and ``oracle`` trains the same program in plain PyTorch without the framework."""
import numpy as np
import torch
from torch import nn


def data_linear(n=64, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(n).astype(np.float32)
    return {"x": x, "y": (3 * x + 2 + 0.1 * rng.randn(n)).astype(np.float32)}


class Linear0(nn.Module):
    def __init__(self):
        super().__init__()
        self.W = nn.Parameter(torch.zeros(()))
        self.b = nn.Parameter(torch.zeros(()))

    def forward(self, x, y):
        return ((self.W * x + self.b - y) ** 2).mean()


class SmallCNN(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(1, 4, 3)
        self.fc1 = nn.Linear(4 * 3 * 3, 6)
        self.fc2 = nn.Linear(6, 3)

    def forward(self, x, y):
        h = torch.relu(self.conv(x))
        h = torch.nn.functional.max_pool2d(h, 2).flatten(1)
        return torch.nn.functional.cross_entropy(self.fc2(torch.relu(self.fc1(h))), y)


class SparseNet(nn.Module):
    """Embedding (row-sparse gradient) -> mean pool -> small MLP, the sentiment-classifier shape."""

    def __init__(self, sparse=True):
        super().__init__()
        self.emb = nn.Embedding(30, 6, sparse=sparse)
        self.fc1 = nn.Linear(6, 6)
        self.fc2 = nn.Linear(6, 1)

    def forward(self, ids, y):
        h = self.emb(ids).mean(1)
        return ((self.fc2(torch.relu(self.fc1(h))).squeeze(-1) - y) ** 2).mean()


class UnrolledLSTM(nn.Module):
    """Two stacked LSTM cells unrolled over time with nested Python loops and a running state (the reference's
    while-loop and dynamic-LSTM cases c4 / c6): the tracer records every iteration as straight-line graph nodes."""

    def __init__(self, steps=5):
        super().__init__()
        self.cells = nn.ModuleList([nn.LSTMCell(3, 6), nn.LSTMCell(6, 6)])
        self.peep = nn.Parameter(torch.full((6,), 0.1))
        self.head = nn.Linear(6, 1)
        self.steps = steps

    def forward(self, x, y):
        B = x.shape[0]
        state = [(x.new_zeros(B, 6), x.new_zeros(B, 6)) for _ in self.cells]
        total = x.new_zeros(B)
        t = 0
        while t < self.steps:                         # python control flow over a static trip count
            inp = x[:, t]
            for li, cell in enumerate(self.cells):
                h, c = cell(inp, state[li])
                h = h + self.peep * torch.tanh(c)     # peephole-like use of the cell state
                state[li] = (h, c)
                inp = h
            total = total + self.head(inp).squeeze(-1)
            t += 1
        return ((total / self.steps - y) ** 2).mean()


def _seq_data(n=8, seed=3):
    rng = np.random.RandomState(seed)
    return {"x": rng.randn(n, 5, 3).astype(np.float32), "y": rng.randn(n).astype(np.float32)}


def _cnn_data(n=8, seed=1):
    rng = np.random.RandomState(seed)
    return {"x": rng.randn(n, 1, 8, 8).astype(np.float32), "y": rng.randint(0, 3, size=n).astype(np.int64)}


def _sparse_data(n=8, seed=2):
    rng = np.random.RandomState(seed)
    return {"ids": rng.randint(0, 30, size=(n, 5)).astype(np.int64), "y": rng.randn(n).astype(np.float32)}


CASES = {
    # name: (model factory, oracle-model factory, data fn, placeholder specs, optimizer factory, steps)
    "c0": (Linear0, Linear0, data_linear, {"x": ((None,), torch.float32), "y": ((None,), torch.float32)},
           lambda ps: torch.optim.SGD(ps, lr=0.01), 5),
    "c1": (SmallCNN, SmallCNN, _cnn_data,
           {"x": ((None, 1, 8, 8), torch.float32), "y": ((None,), torch.int64)},
           lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9), 4),
    "c2": (lambda: SparseNet(True), lambda: SparseNet(False), _sparse_data,
           {"ids": ((None, 5), torch.int64), "y": ((None,), torch.float32)},
           lambda ps: torch.optim.Adagrad(ps, lr=0.1), 4),
    "c3": (lambda: SparseNet(True), lambda: SparseNet(False), _sparse_data,
           {"ids": ((None, 5), torch.int64), "y": ((None,), torch.float32)},
           lambda ps: torch.optim.Adam(ps, lr=0.01), 4),
    "c4": (UnrolledLSTM, UnrolledLSTM, _seq_data,
           {"x": ((None, 5, 3), torch.float32), "y": ((None,), torch.float32)},
           lambda ps: torch.optim.SGD(ps, lr=0.1, momentum=0.5), 4),
}


def oracle(case, seed=7):
    _, factory, data_fn, _, opt_fn, steps = CASES[case]
    torch.manual_seed(seed)
    model = factory()
    opt = opt_fn(list(model.parameters()))
    data = {k: torch.from_numpy(v) for k, v in data_fn().items()}
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(**data)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return {k: v.detach().clone() for k, v in model.state_dict().items()}, losses
