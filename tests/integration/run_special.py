"""Multi-rank scenarios that are not plain strategy x case runs: self-launch through the coordinator,
bounded staleness, asynchronous PS, worker failure, cross-strategy checkpoint reload, ad.function."""
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from autodist_b200 import AutoDist  # noqa: E402
from autodist_b200.autodist import _reset_default_autodist  # noqa: E402
from autodist_b200.checkpoint.saver import Saver  # noqa: E402
from autodist_b200.resource_spec import ResourceSpec  # noqa: E402
from autodist_b200.strategy import PS, AllReduce, PartitionedPS  # noqa: E402
import cases  # noqa: E402


def build(ad, case="c0"):
    factory, _, data_fn, ph_specs, opt_fn, steps = cases.CASES[case]
    torch.manual_seed(7)
    model = factory()
    phs = {k: ad.placeholder(shape, dtype, name=k) for k, (shape, dtype) in ph_specs.items()}
    loss = model(**phs)
    opt = opt_fn(list(model.parameters()))
    return model, phs, loss, opt.minimize(loss), data_fn()


def scenario_selflaunch():
    """No external launcher: the chief re-executes this script for the second replica."""
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=AllReduce(chunk_size=4))
    ref_state, _ = cases.oracle("c0")
    with ad.scope():
        model, phs, loss, train_op, data = build(ad)
        sess = ad.create_distributed_session()
        for _ in range(5):
            sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
        w = sess.run(model.W)
    assert abs(float(w) - float(ref_state["W"])) < 1e-5, (w, ref_state["W"])
    print(f"selflaunch rank {sess.rank} ok", flush=True)


def scenario_stale():
    """staleness=2: the fast rank never leads by more than 2 steps, and it does get ahead."""
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=PS(sync=True, staleness=2))
    with ad.scope():
        model, phs, loss, train_op, data = build(ad)
        sess = ad.create_distributed_session()
        leads = []
        for step in range(8):
            if sess.rank == 1:
                time.sleep(0.3)   # the slow worker
            sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
            leads.append(sess.engine._async.last_lead)
        lv = sess.run(loss, {phs[k]: data[k] for k in phs})
    assert max(leads) <= 2, leads
    if sess.rank == 0:
        assert max(leads) >= 1, f"the fast rank never ran ahead: {leads}"
    assert np.isfinite(lv)
    print(f"stale rank {sess.rank} leads {leads} ok", flush=True)


def scenario_async():
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=PS(sync=False))
    with ad.scope():
        model, phs, loss, train_op, data = build(ad)
        sess = ad.create_distributed_session()
        first = None
        for step in range(6 if sess.rank == 0 else 3):   # ranks take different numbers of steps: no lock-step
            lv, _ = sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
            first = lv if first is None else first
    assert lv < first
    print(f"async rank {sess.rank} ok", flush=True)


def scenario_failure():
    """A worker that exits with an error surfaces in the chief as WorkerFailure, not as a hang."""
    from autodist_b200.coordinator import WorkerFailure
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=AllReduce())
    with ad.scope():
        model, phs, loss, train_op, data = build(ad)
        sess = ad.create_distributed_session()
        sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
        if sess.rank == 1:
            os._exit(3)       # dies between steps, nothing in flight
        caught = None
        for _ in range(50):
            try:
                time.sleep(0.2)
                sess.run(model.W)        # no collective; the coordinator check raises
            except WorkerFailure as e:
                caught = e
                break
    assert caught is not None
    print("failure surfaced ok:", caught, flush=True)
    os._exit(0)


def scenario_crossload():
    """Save under PartitionedPS, restore under AllReduce in a second session of the same ranks."""
    tmp = os.environ["AUTODIST_TEST_TMP"]
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2),
                  strategy_builder=PartitionedPS(num_shards=2, reduction_devices="gpu"))
    with ad.scope():
        model, phs, loss, train_op, data = build(ad, "c3")
        saver = Saver(max_to_keep=2)
        sess = ad.create_distributed_session()
        for step in range(1, 4):
            sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
            path = saver.save(sess, os.path.join(tmp, "m"), global_step=step)
        after3 = {n: sess.run(n) for n, _ in ad.graph_item.named_parameters()}
        sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
        after4 = {n: sess.run(n) for n, _ in ad.graph_item.named_parameters()}
        sess.close()
    if sess.rank == 0:
        assert not os.path.exists(os.path.join(tmp, "m-1")) and os.path.exists(os.path.join(tmp, "m-3.index"))
        plain = torch.load(path, weights_only=False)
        assert plain["variables"]["emb.weight"].shape == (30, 6)          # merged, original name
        assert plain["slots"]["emb.weight/exp_avg"].shape == (30, 6)      # optimizer slot merged too
        assert plain["slices"]["emb.weight"] == [[[0, 0], [15, 6]], [[15, 0], [15, 6]]]
    _reset_default_autodist()
    ad2 = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=AllReduce(chunk_size=2))
    with ad2.scope():
        torch.manual_seed(99)   # different init: restore must overwrite it
        model, phs, loss, train_op, data = build(ad2, "c3")
        torch.manual_seed(123)
        for p in model.parameters():
            p.data.normal_()
        saver2 = Saver()
        sess2 = ad2.create_distributed_session()
        saver2.restore(sess2, path)
        for n, v in after3.items():
            assert np.allclose(sess2.run(n), v, atol=1e-7), n
        sess2.run([loss, train_op], {phs[k]: data[k] for k in phs})   # continues exactly (Adam slots restored)
        for n, v in after4.items():
            assert np.allclose(sess2.run(n), v, atol=1e-5), (n, np.abs(sess2.run(n) - v).max())
    print(f"crossload rank {sess2.rank} ok", flush=True)


def scenario_function():
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=AllReduce())
    ref_state, ref_losses = cases.oracle("c0")
    data = cases.data_linear()
    with ad.scope():
        torch.manual_seed(7)
        model = cases.Linear0()
        opt = torch.optim.SGD(model.parameters(), lr=0.01)

        @ad.function
        def train_step(x, y):
            loss = model(x, y)
            return loss, opt.minimize(loss), model.b

        for _ in range(5):
            loss, _, b = train_step(data["x"], y=data["y"])
    assert abs(float(b) - float(ref_state["b"])) < 1e-5
    print(f"function rank {ad.rank} ok", flush=True)


TWO_NODE_SPEC = """
nodes:
  - address: 10.0.0.1
    cpus: [0, 1]
    chief: true
  - address: 10.0.0.2
    cpus: [0, 1]
    ssh_config: conf
ssh:
  conf:
    username: nobody
"""


def _run_multi_node(tag, spec_text, world, local_ranks_of, case="c1"):
    tmp = os.environ["AUTODIST_TEST_TMP"]
    path = os.path.join(tmp, f"{tag}_{os.environ['RANK']}.yml")
    with open(path, "w") as f:
        f.write(spec_text)
    results = {}
    for name, builder in (("AllReduce", AllReduce(chunk_size=1)), ("PartitionedPS", PartitionedPS()), ("PS", PS())):
        _reset_default_autodist()
        ad = AutoDist(resource_spec_file=path, strategy_builder=builder)
        ref_state, _ = cases.oracle(case)
        with ad.scope():
            model, phs, loss, train_op, data = build(ad, case)
            sess = ad.create_distributed_session()
            info = sess.engine.plan.replica
            assert info.world_size == world and info.num_workers == 2
            assert info.local_ranks == local_ranks_of(sess.rank), info.local_ranks
            for _ in range(4):
                sess.run([loss, train_op], {phs[k]: data[k] for k in phs})
            got = {n: sess.run(p) for n, p in model.named_parameters()}
            sess.close()
        diff = max(float(np.abs(got[n] - ref_state[n].numpy()).max()) for n in got)
        assert diff < 1e-5, (name, diff)
        results[name] = diff
    print(f"{tag} {case} rank {os.environ['RANK']} ok {results}", flush=True)


def scenario_twonode():
    """A two-node resource spec (two replicas per node) run as four externally launched ranks on one host: ranks 0-1
    form node 10.0.0.1, ranks 2-3 node 10.0.0.2. Every process feeds its node's batch, which is split between the two
    replicas of that node; a hierarchical plan (two workers) must still equal the single-process run."""
    _run_multi_node("twonode", TWO_NODE_SPEC, 4, lambda r: [0, 1] if r < 2 else [2, 3])
    # row-sparse embedding + Adagrad: sparse rows are gathered across both nodes, owners publish the touched rows
    _run_multi_node("twonode", TWO_NODE_SPEC, 4, lambda r: [0, 1] if r < 2 else [2, 3], case="c2")


def scenario_hetero():
    """Nodes of different size (two replicas and one, the shape of the reference's r4 spec): the lone replica of the
    second node takes that node's whole batch."""
    spec = TWO_NODE_SPEC.replace("    cpus: [0, 1]\n    ssh_config: conf", "    cpus: [0]\n    ssh_config: conf")
    assert spec != TWO_NODE_SPEC
    _run_multi_node("hetero", spec, 3, lambda r: [0, 1] if r < 2 else [2])


def scenario_twoopts():
    """Two optimizers over disjoint variables, both train ops fetched by one run() on two replicas: the result equals the
    single-process computation on the whole batch (gradients of both losses taken at the values before the step)."""
    import copy
    torch.manual_seed(2)
    enc0, head0 = torch.nn.Linear(5, 4), torch.nn.Linear(4, 1)
    g = torch.Generator().manual_seed(0)
    data = [(torch.randn(8, 5, generator=g), torch.randn(8, 1, generator=g)) for _ in range(4)]
    enc, head = copy.deepcopy(enc0), copy.deepcopy(head0)
    o1, o2 = torch.optim.SGD(enc.parameters(), lr=0.1), torch.optim.Adam(head.parameters(), lr=0.01)
    for xb, yb in data:
        h = torch.tanh(enc(xb))
        l1, l2 = (h ** 2).mean(), ((head(h) - yb) ** 2).mean()
        o1.zero_grad()
        o2.zero_grad()
        l1.backward(inputs=list(enc.parameters()), retain_graph=True)
        l2.backward(inputs=list(head.parameters()))
        o1.step()
        o2.step()
    strategy = PS() if os.environ.get("AUTODIST_TWOOPTS", "ar") == "ps" else AllReduce(chunk_size=2)
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=2), strategy_builder=strategy)
    with ad.scope():
        e, hd = copy.deepcopy(enc0), copy.deepcopy(head0)
        x = ad.placeholder((None, 5), torch.float32, name="x")
        y = ad.placeholder((None, 1), torch.float32, name="y")
        hidden = torch.tanh(e(x))
        loss1, loss2 = (hidden ** 2).mean(), ((hd(hidden) - y) ** 2).mean()
        op1 = torch.optim.SGD(e.parameters(), lr=0.1).minimize(loss1, var_list=list(e.parameters()))
        op2 = torch.optim.Adam(hd.parameters(), lr=0.01).minimize(loss2, var_list=list(hd.parameters()))
        sess = ad.create_distributed_session()
        for xb, yb in data:
            sess.run([loss1, loss2, op1, op2], {x: xb, y: yb})
        got = [sess.run(p) for p in list(e.parameters()) + list(hd.parameters())]
    want = [p.detach().numpy() for p in list(enc.parameters()) + list(head.parameters())]
    for a, b in zip(got, want):
        assert np.allclose(a, b, atol=2e-5), (a, b)
    print(f"twoopts rank {sess.rank} ok", flush=True)


def _spawn_ranks(name, nproc=2):
    """Start the ranks the way an external launcher would (RANK / WORLD_SIZE in the environment)."""
    import subprocess
    port = 21000 + (os.getpid() % 20000)
    procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), name],
                              env=dict(os.environ, RANK=str(r), WORLD_SIZE=str(nproc), LOCAL_RANK=str(r),
                                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port)))
             for r in range(nproc)]
    codes = [p.wait(timeout=500) for p in procs]
    sys.exit(0 if all(c == 0 for c in codes) else 1)


if __name__ == "__main__":
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)
    if sys.argv[1] in ("crossload", "twonode", "hetero") and "RANK" not in os.environ:
        _spawn_ranks(sys.argv[1], {"twonode": 4, "hetero": 3}.get(sys.argv[1], 2))
    globals()["scenario_" + sys.argv[1]]()
