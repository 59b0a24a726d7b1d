"""Data-dependent control flow in captured programs (the reference's tf.cond / tf.while_loop cases,
tests/integration/cases/c2.py:50-52 and c4.py:31): a module whose forward branches or loops on tensor values is recorded as one
opaque node, its variables are marked ``in_control_flow``, and the partitioning builders leave them whole."""
import pytest
import torch
from torch import nn

from autodist_b200 import AutoDist
from autodist_b200.autodist import _reset_default_autodist
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200 import strategy as S


class GuardedEmbedding(nn.Module):
    """An embedding looked up only when the ids are non-negative (the guard of the reference's case c2)."""

    def __init__(self):
        super().__init__()
        self.table = nn.Parameter(torch.randn(12, 4))
        self.fallback = nn.Parameter(torch.zeros(4))

    def forward(self, ids):
        if bool((ids >= 0).all()):
            return self.table[ids]
        return self.fallback.expand(ids.shape[0], 4)


class Repeat(nn.Module):
    """Applies ``tanh(x w)`` until the norm drops below a bound (a while loop on a tensor value, the reference's case c4)."""

    def __init__(self):
        super().__init__()
        self.w = nn.Parameter(torch.full((4, 4), 0.5))

    def forward(self, x):
        steps = 0
        while float(x.detach().norm()) > 1.0 and steps < 4:
            x = torch.tanh(x @ self.w)
            steps += 1
        return x


def _build(builder):
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=0), strategy_builder=builder)
    with ad.scope():
        torch.manual_seed(0)
        emb, rep, head = GuardedEmbedding(), Repeat(), nn.Linear(4, 1)
        ids = ad.placeholder((None,), torch.int64, name="ids")
        loss = head(rep(emb(ids))).pow(2).mean()
        train_op = torch.optim.SGD(list(emb.parameters()) + list(rep.parameters()) + list(head.parameters()), lr=0.01).minimize(loss)
        sess = ad.create_distributed_session()
    return ad, sess, ids, loss, train_op, (emb, rep, head)


def test_modules_with_data_dependent_control_flow_run_as_opaque_nodes():
    ad, sess, ids, loss, train_op, (emb, rep, head) = _build(S.PS())
    item = ad.graph_item
    flags = {v.name: v.in_control_flow for v in item.variables.values()}
    assert flags["guardedembedding/table:0"] and flags["guardedembedding/fallback:0"] and flags["repeat/w:0"]
    assert not flags["linear/weight:0"] and not flags["linear/bias:0"]
    kinds = [n.op for n in item.tracer.graph.nodes]
    assert kinds.count("call_module") >= 2                     # the two control-flow modules are single nodes
    feed = {ids: torch.tensor([1, 2, 3, 4])}
    first = float(sess.run([loss, train_op], feed)[0])
    for _ in range(5):
        last = float(sess.run([loss, train_op], feed)[0])
    assert last < first
    # the other branch of the guard runs too (decided per call, at run time)
    other = float(sess.run(loss, {ids: torch.tensor([-1, 2, 3, 4])}))
    assert other == other
    sess.close()


@pytest.mark.parametrize("builder", [lambda: S.PartitionedPS(), lambda: S.UnevenPartitionedPS(),
                                     lambda: S.PartitionedAR(), lambda: S.RandomAxisPartitionAR()])
def test_control_flow_variables_are_never_partitioned(builder):
    ad, sess, ids, loss, train_op, _ = _build(builder())
    plan = sess.engine.plan
    guarded = ("guardedembedding/table:0", "guardedembedding/fallback:0", "repeat/w:0")
    for name in guarded:
        assert name not in plan.shard_plans or plan.shard_plans[name].num_shards == 1, (name, plan.shard_plans[name])
    parts = [e.part for e in plan.ps_entries.values()] + [p for b in plan.ordered_buckets() for p in b.parts]
    assert all(p.part_index is None for p in parts if p.var_name in guarded)
    sess.run([loss, train_op], {ids: torch.tensor([0, 5, 7, 11])})
    sess.close()


def test_control_flow_written_directly_in_the_scope_is_refused_with_a_hint():
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=0), strategy_builder=S.PS())
    with ad.scope():
        x = ad.placeholder((None, 3), torch.float32, name="x")
        with pytest.raises(Exception, match="nn.Module"):
            if x.sum() > 0:
                pass
