"""Graph capture: optimizer sweep, sparse detection, default-item context, proto round trip."""
import pytest
import torch
from torch import nn

from autodist_b200 import graph_item as gi
from autodist_b200.graph_item import GraphItem

gi.patch_optimizers()

OPTIMIZERS = [
    (torch.optim.SGD, dict(lr=0.1)), (torch.optim.SGD, dict(lr=0.1, momentum=0.9)),
    (torch.optim.SGD, dict(lr=0.1, momentum=0.9, nesterov=True)), (torch.optim.Adam, dict(lr=1e-3)),
    (torch.optim.Adam, dict(lr=1e-3, amsgrad=True)), (torch.optim.AdamW, dict(lr=1e-3)),
    (torch.optim.Adagrad, dict(lr=0.1)), (torch.optim.RMSprop, dict(lr=0.01)),
    (torch.optim.RMSprop, dict(lr=0.01, centered=True, momentum=0.5)), (torch.optim.Adadelta, dict()),
    (torch.optim.Adamax, dict()), (torch.optim.NAdam, dict()), (torch.optim.RAdam, dict()),
    (torch.optim.ASGD, dict()),
]


class Net(nn.Module):
    def __init__(self, sparse):
        super().__init__()
        self.emb = nn.Embedding(50, 8, sparse=sparse)
        self.fc = nn.Linear(8, 1)

    def forward(self, ids):
        return self.fc(self.emb(ids).mean(1))


@pytest.mark.parametrize("cls,kw", OPTIMIZERS)
def test_optimizer_capture(cls, kw):
    item = GraphItem()
    with item.as_default():
        net = Net(sparse=False)
        ids = item.placeholder((None, 4), torch.int64, name="ids")
        y = item.placeholder((None, 1), torch.float32, name="y")
        loss = ((net(ids) - y) ** 2).mean()
        opt = cls(net.parameters(), **kw)
        op = opt.minimize(loss)
    item.prepare()
    assert item.optimizers[0].cls is cls
    trainables = item.trainable_var_op_to_var
    assert set(trainables) == {"emb.weight", "fc.weight", "fc.bias"}
    info = item.var_op_name_to_grad_info
    assert len(info) == len(trainables)
    assert info["fc.weight"][0] == "gradients/fc.weight_grad:0"
    assert op.loss_node.name == "mean_1" or op.loss_node.op == "call_method"


def test_sparse_detection_and_pruning():
    item = GraphItem()
    with item.as_default():
        net = Net(sparse=True)
        unused = nn.Linear(3, 3)
        ids = item.placeholder((None, 4), torch.int64)
        loss = net(ids).sum()
        opt = torch.optim.SGD(list(net.parameters()) + list(unused.parameters()), lr=0.1)
        opt.minimize(loss)
    item.prepare()
    v = item.variables
    assert v["net/emb.weight:0"].sparse_grad and not v["net/fc.weight:0"].sparse_grad
    # the unused layer has no path to the loss: it has no update
    assert "linear/weight:0" in v and "linear/weight:0" not in item.updated_variable_names()


def test_default_item_not_nestable():
    a, b = GraphItem(), GraphItem()
    with a.as_default():
        assert gi.get_default_graph_item() is a
        with pytest.raises(SyntaxError):
            with b.as_default():
                pass
    assert gi.get_default_graph_item() is None


def test_bare_variables_and_round_trip():
    item = GraphItem()
    with item.as_default():
        w = item.variable(0.0, name="W")
        b = item.variable(0.0, name="b")
        x = item.placeholder((None,), name="x")
        loss = ((w * x + b) ** 2).mean()
        torch.optim.SGD([w, b], lr=0.1).minimize(loss)
    item.prepare()
    assert list(item.trainable_var_op_to_var) == ["W", "b"]
    data = item.serialize()
    again = GraphItem.deserialize(data)
    assert again == item
    assert again.grad_target_pairs == {"gradients/W_grad:0": "W:0", "gradients/b_grad:0": "b:0"}
    assert again.variables["W:0"].shape == ()


def test_leaf_module_is_one_node():
    class Whole(nn.Module):
        _autodist_leaf = True

        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(4, 2)

        def forward(self, x):
            return self.fc(x).sum() if x.shape[0] > 0 else x.sum()   # data-dependent python: not traceable

    item = GraphItem()
    with item.as_default():
        m = Whole()
        x = item.placeholder((None, 4))
        loss = m(x)
        torch.optim.SGD(m.parameters(), lr=0.1).minimize(loss)
    assert [n.op for n in item.tracer.graph.nodes] == ["placeholder", "call_module"]
    assert item.updated_variable_names() == {"fc.weight:0", "fc.bias:0"}


def test_captured_optimizer_arguments_rebuild_the_same_optimizer_class():
    """The recorded constructor arguments must be accepted by the optimizer's own class (AdamW passes its parent an argument
    it does not take itself), and groups keep their own hyper-parameters."""
    import torch
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1))
    with ad.scope():
        a, b = torch.nn.Parameter(torch.zeros(2)), torch.nn.Parameter(torch.zeros(3))
        for cls in (torch.optim.AdamW, torch.optim.Adam, torch.optim.SGD, torch.optim.Adagrad, torch.optim.RMSprop):
            opt = cls([{"params": [a], "weight_decay": 0.5}, {"params": [b], "lr": 0.25}], lr=0.125)
            info = ad.graph_item.optimizers[-1]
            again = info.cls([{"params": [torch.nn.Parameter(torch.zeros(2))]}], **dict(info.kwargs))
            assert type(again) is cls and again.defaults["lr"] == 0.125
            assert opt.param_groups[0]["weight_decay"] == 0.5 and opt.param_groups[1]["lr"] == 0.25
    _reset_default_autodist()
