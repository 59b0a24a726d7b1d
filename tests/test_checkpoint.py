"""Checkpoints written under a distributed strategy load in plain PyTorch (original names, partitions merged), resume
training exactly, rotate, and export as a saved model (reference: ``tests/checkpoint/test_keras_saver.py``,
``test_partitionedPS_saver.py``, ``test_saved_model.py``)."""
import json
import os

import pytest
import torch
from torch import nn

from autodist_b200 import AutoDist
from autodist_b200.autodist import _reset_default_autodist
from autodist_b200.checkpoint.saved_model_builder import SavedModelBuilder, load_saved_model
from autodist_b200.checkpoint.saver import Saver, latest_checkpoint
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200 import strategy as S


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(101, 8, sparse=True)        # 101 rows: prime, so PartitionedPS uses 101 one-row shards
        self.fc = nn.Linear(8, 1)

    def forward(self, ids, y):
        return ((self.fc(self.emb(ids).mean(1)).squeeze(-1) - y) ** 2).mean()


def _data():
    g = torch.Generator().manual_seed(0)
    return {"ids": torch.randint(0, 101, (16, 4), generator=g), "y": torch.randn(16, generator=g)}


def _session(builder, seed=3, max_to_keep=5):
    _reset_default_autodist()
    os.environ["AUTODIST_IS_TESTING"] = "True"               # allows partitioning with a single parameter server
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=builder)
    data = _data()
    scope = ad.scope()
    scope.__enter__()
    torch.manual_seed(seed)
    model = Net()
    phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in data.items()}
    loss = model(**phs)
    train_op = torch.optim.Adagrad(model.parameters(), lr=0.1).minimize(loss)
    saver = Saver(max_to_keep=max_to_keep)
    sess = ad.create_distributed_session()

    def step():
        return float(sess.run([loss, train_op], {phs[k]: data[k] for k in phs})[0])

    def done():
        sess.close()
        scope.__exit__(None, None, None)
        _reset_default_autodist()
        os.environ.pop("AUTODIST_IS_TESTING", None)

    return ad, sess, saver, step, done


def test_partitioned_checkpoint_loads_in_plain_pytorch_and_resumes(tmp_path):
    ad, sess, saver, step, done = _session(S.PartitionedPS())
    parts = [n for n in ad.strategy.node_config if n.var_name.startswith("emb")][0]
    assert len(parts.part_config) > 1                        # the table really is sharded
    for _ in range(3):
        step()
    path = saver.save(sess, str(tmp_path / "ckpt" / "model"), global_step=3)
    assert path.endswith("model-3") and latest_checkpoint(str(tmp_path / "ckpt")) == path
    expected_next = [step() for _ in range(2)]
    done()
    # plain PyTorch: no framework objects needed to read the file
    state = torch.load(path, map_location="cpu", weights_only=False)
    assert state["variables"]["emb.weight"].shape == (101, 8)              # merged under the original name
    assert len(state["slices"]["emb.weight"]) == len(parts.part_config)
    assert state["slots"]["emb.weight/sum"].shape == (101, 8)
    plain = Net()
    plain.load_state_dict(state["variables"])
    opt = torch.optim.Adagrad(plain.parameters(), lr=0.1)
    opt_state = {i: {"sum": state["slots"][f"{n}/sum"].clone(), "step": torch.tensor(3.0)}
                 for i, (n, _) in enumerate(plain.named_parameters())}
    opt.load_state_dict({"state": opt_state, "param_groups": opt.state_dict()["param_groups"]})
    data = _data()
    got = []
    for _ in range(2):
        opt.zero_grad()
        loss = plain(**data)
        loss.backward()
        plain.emb.weight.grad = plain.emb.weight.grad.coalesce()
        opt.step()
        got.append(float(loss.detach()))
    assert got == pytest.approx(expected_next, rel=1e-5)
    # restore under a different strategy continues identically
    ad, sess, saver, step, done = _session(S.AllReduce(), seed=99)
    saver.restore(sess, path)
    assert [step() for _ in range(2)] == pytest.approx(expected_next, rel=1e-5)
    done()


def test_rotation_keeps_the_newest_checkpoints(tmp_path):
    ad, sess, saver, step, done = _session(S.PS(), max_to_keep=2)
    base = str(tmp_path / "model")
    paths = []
    for i in range(4):
        step()
        paths.append(saver.save(sess, base, global_step=i))
    done()
    assert [os.path.exists(p) for p in paths] == [False, False, True, True]
    with open(tmp_path / "checkpoint") as f:
        rec = json.load(f)
    assert rec["model_checkpoint_path"] == "model-3" and rec["all_model_checkpoint_paths"] == ["model-2", "model-3"]
    assert os.path.exists(paths[-1] + ".index") and os.path.exists(paths[-1] + ".meta")


def test_saver_must_precede_the_session():
    ad, sess, saver, step, done = _session(S.PS())
    with pytest.raises(RuntimeError):
        Saver()
    done()


def test_saved_model_export_and_reload(tmp_path):
    ad, sess, saver, step, done = _session(S.PSLoadBalancing())
    for _ in range(2):
        step()
    export = str(tmp_path / "export")
    builder = SavedModelBuilder(export)
    with pytest.raises(ValueError):
        builder.add_meta_graph_and_variables(sess, ["serve"], saver=None)
    builder.add_meta_graph_and_variables(sess, ["serve", "train"], saver=saver)
    assert builder.save() == export
    next_loss = step()
    done()
    meta, state = load_saved_model(export)
    assert meta["tags"] == ["serve", "train"] and len(meta["train_ops"]) == 1
    assert {p["name"] for p in meta["placeholders"]} == {"ids", "y"} and meta["strategy_id"]
    assert "emb" in meta["graph"]
    with pytest.raises(AssertionError):
        SavedModelBuilder(export)                            # refuses a non-empty directory
    # continue training from the export in a fresh process state
    ad, sess, saver, step, done = _session(S.PS(), seed=1234)
    saver.restore(sess, os.path.join(export, meta["variables"]))
    assert step() == pytest.approx(next_loss, rel=1e-5)
    done()
