"""Training-loop utilities, the NeuMF model and BERT config IO (CPU)."""
import io
import json

import pytest
import torch

from autodist_b200.utils import train_utils as tu


def test_time_history_windows():
    t = iter([0.0, 1.0, 3.0, 4.0])
    h = tu.TimeHistory(batch_size=10, log_steps=2, clock=lambda: next(t))
    h.on_train_begin()
    recs = [h.on_step_end() for _ in range(6)]
    assert [r is not None for r in recs] == [False, True, False, True, False, True]
    assert recs[1] == {"step": 2, "elapsed_s": 1.0, "examples_per_sec": 20.0}
    assert recs[3]["examples_per_sec"] == 10.0
    assert h.average_examples_per_sec == pytest.approx((10.0 + 20.0) / 2)


def test_metrics_logger_writes_jsonl(tmp_path):
    path = tmp_path / "m" / "metrics.jsonl"
    buf = io.StringIO()
    lg = tu.MetricsLogger(str(path), stream=buf)
    lg.log_run_info("bert", "synthetic", {"batch": 32})
    assert lg.log_metric("loss", torch.tensor(1.5), "nats", 3)
    assert not lg.log_metric("bad", "not a number")
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["kind"] for r in rows] == ["run_info", "metric"]
    assert rows[1]["value"] == 1.5 and rows[1]["global_step"] == 3
    assert len(buf.getvalue().splitlines()) == 2


def test_learning_rate_schedules():
    assert tu.warmup_linear_decay(0, 1.0, 100, 10) == pytest.approx(0.1)
    assert tu.warmup_linear_decay(10, 1.0, 100, 10) == pytest.approx(1.0)
    assert tu.warmup_linear_decay(55, 1.0, 100, 10) == pytest.approx(0.5)
    assert tu.warmup_linear_decay(1000, 1.0, 100, 10) == 0.0
    sched = tu.PiecewiseConstantDecayWithWarmup(batch_size=512, epoch_size=5120, warmup_epochs=5, boundaries=[30, 60, 80, 90],
                                                multipliers=[1.0, 0.1, 0.01, 0.001, 0.0001])
    assert sched.rescaled_lr == pytest.approx(0.2) and sched.steps_per_epoch == 10
    assert sched(0) == 0.0 and sched(25) == pytest.approx(0.1) and sched(50) == pytest.approx(0.2)
    assert sched(300) == pytest.approx(0.02) and sched(950) == pytest.approx(0.2e-4)
    with pytest.raises(ValueError):
        tu.PiecewiseConstantDecayWithWarmup(256, 1000, 1, [1, 2], [1.0, 0.1])
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=torch.tensor(0.5))
    tu.set_learning_rate(opt, 0.25)
    assert float(opt.param_groups[0]["lr"]) == 0.25


def test_flag_groups_and_strategy_switch():
    import argparse
    from autodist_b200 import strategy as S
    ap = argparse.ArgumentParser()
    tu.add_base_flags(ap)
    tu.add_performance_flags(ap)
    tu.add_benchmark_flags(ap)
    tu.add_strategy_flags(ap)
    a = ap.parse_args(["--autodist_strategy", "Parallax", "--chunk_size", "64", "--compressor", "HorovodCompressorEF"])
    assert a.batch_size == 32 and a.log_steps == 100 and a.dtype == "bf16"
    b = tu.build_strategy(a.autodist_strategy, a.chunk_size, a.compressor)
    assert isinstance(b, S.Parallax)
    for name in ["PS", "PSLoadBalancing", "PartitionedPS", "UnevenPartitionedPS", "AllReduce", "PartitionedAR",
                 "RandomAxisPartitionAR", "Auto"]:
        assert tu.build_strategy(name) is not None
    with pytest.raises(ValueError):
        tu.build_strategy("nope")


def test_bert_config_json_round_trip(tmp_path):
    from autodist_b200.models.bert import BertConfig
    cfg = BertConfig.base(hidden_dropout_prob=0.0)
    p = tmp_path / "bert_config.json"
    obj = json.loads(cfg.to_json_string())
    obj["hidden_act"] = "gelu"                         # keys of published files that this model fixes are ignored
    p.write_text(json.dumps(obj))
    assert BertConfig.from_json_file(str(p)) == cfg


def test_neumf_metrics_and_sparse_gradients():
    from autodist_b200.models.ncf import NeuMF, NeuMFConfig, hit_rate_and_ndcg, synthetic_interactions
    cfg = NeuMFConfig.tiny()
    torch.manual_seed(0)
    m = NeuMF(cfg)
    d = synthetic_interactions(40, cfg)
    assert d["labels"].sum() == 8
    m(**d).backward()
    assert m.user_emb.grad.is_sparse and m.item_emb.grad.is_sparse
    md = NeuMF(NeuMFConfig.tiny(dense_gradient=True))
    md.load_state_dict(m.state_dict())
    md(**d).backward()
    assert not md.user_emb.grad.is_sparse
    torch.testing.assert_close(md.user_emb.grad, m.user_emb.grad.to_dense())
    w = torch.zeros(40)
    w[:5] = 1
    full = torch.nn.functional.binary_cross_entropy_with_logits(m.logits(d["users"][:5], d["items"][:5]), d["labels"][:5])
    torch.testing.assert_close(m(d["users"], d["items"], d["labels"], w), full)
    scores = torch.tensor([[5.0, 1.0, 2.0], [0.0, 1.0, 2.0], [1.5, 1.0, 2.0]])
    hr, ndcg = hit_rate_and_ndcg(scores, top_k=2)
    assert hr == pytest.approx(2 / 3)
    assert ndcg == pytest.approx((1.0 + 0.0 + 1.0 / torch.log2(torch.tensor(3.0)).item()) / 3)
    with pytest.raises(ValueError):
        NeuMF(NeuMFConfig(10, 10, 4, [7, 4]))
