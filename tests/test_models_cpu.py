"""Every model family trains through the public API on CPU (single replica, tiny configurations)."""
import numpy as np
import pytest
import torch

from autodist_b200 import AutoDist
from autodist_b200.autodist import _reset_default_autodist
from autodist_b200.resource_spec import ResourceSpec
from autodist_b200 import strategy as S


def _train(model_fn, data, opt_fn, builder, steps=4, clip=None):
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=builder)
    with ad.scope():
        torch.manual_seed(0)
        model = model_fn()
        phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in data.items()}
        loss = model(**phs)
        opt = opt_fn(model)
        train_op = opt.minimize(loss, clip_global_norm=clip(model) if clip else None)
        sess = ad.create_distributed_session()
        losses = [float(sess.run([loss, train_op], {phs[k]: data[k] for k in phs})[0]) for _ in range(steps)]
        sess.close()
    _reset_default_autodist()
    assert all(np.isfinite(losses)), losses
    return losses


def test_bert_tiny_reference_path():
    from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch
    cfg = BertConfig.tiny()
    losses = _train(lambda: BertPretrainer(cfg), synthetic_batch(cfg, 4, 32, 4),
                    lambda m: torch.optim.Adam(m.parameters(), lr=1e-3), S.Parallax(), steps=5)
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("backbone,size", [("resnet50", 32), ("vgg16", 32), ("densenet121", 32), ("inceptionv3", 96)])
def test_cnn_families(backbone, size):
    from autodist_b200.models.cnn import ImageClassifier, synthetic_images
    kw = {"image_size": size} if backbone == "vgg16" else {}
    losses = _train(lambda: ImageClassifier(backbone, num_classes=10, **kw), synthetic_images(4, size, 10),
                    lambda m: torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9), S.AllReduce(chunk_size=25), steps=3)
    assert len(losses) == 3


def test_lm1b_tiny_with_clipping():
    from autodist_b200.models.lm1b import LM1B, LM1BConfig, zipf_tokens
    cfg = LM1BConfig.tiny()
    losses = _train(lambda: LM1B(cfg), zipf_tokens(8, cfg.num_steps, cfg.vocab_size),
                    lambda m: torch.optim.Adagrad(m.parameters(), lr=0.2, initial_accumulator_value=1.0),
                    S.PartitionedPS(), steps=16, clip=lambda m: (cfg.max_grad_norm, m.dense_parameters()))
    assert min(losses[8:]) < losses[0]      # negatives are re-sampled every step: compare the trend, not neighbours


def test_small_models():
    from autodist_b200.models.simple import FashionCNN, NeuMF, SentimentClassifier
    rng = np.random.RandomState(0)
    d = {"images": torch.rand(8, 1, 28, 28), "labels": torch.randint(0, 10, (8,))}
    _train(FashionCNN, d, lambda m: torch.optim.SGD(m.parameters(), lr=0.05), S.PSLoadBalancing())
    d = {"ids": torch.randint(0, 10000, (8, 16)), "labels": torch.randint(0, 2, (8,)).float()}
    _train(SentimentClassifier, d, lambda m: torch.optim.Adagrad(m.parameters(), lr=0.2), S.PartitionedPS())
    d = {"users": torch.randint(0, 50, (16,)), "items": torch.randint(0, 40, (16,)), "labels": torch.randint(0, 2, (16,)).float()}
    _train(lambda: NeuMF(50, 40, 8, (16, 16, 8)), d, lambda m: torch.optim.SGD(m.parameters(), lr=0.1), S.Parallax())
