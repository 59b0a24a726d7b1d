"""Host-to-device staging of fed values: a queued copy must never read a batch the host has already replaced."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_staging_buffers_are_not_overwritten_while_a_copy_is_queued():
    from autodist_b200.remapper import PinnedStager
    dev = torch.device("cuda", 0)
    stager = PinnedStager(dev)
    a = torch.randn(4096, 4096, device=dev)
    batches = [torch.full((1 << 20,), float(i)) for i in range(8)]          # ordinary (pageable) host tensors
    # keep the stream busy so that the uploads below queue up behind it, as they do behind a replayed step
    for _ in range(20):
        a = a @ a * 1e-3
    got = [stager.upload("x", b) for b in batches]
    torch.cuda.synchronize()
    for i, g in enumerate(got):
        assert float(g.min()) == float(i) and float(g.max()) == float(i), f"batch {i} arrived as {float(g.min())}..{float(g.max())}"


def test_feeds_of_consecutive_steps_reach_the_model_without_a_tensor_fetch():
    """Distinct unpinned batches, only ``train_op`` fetched (nothing synchronises the host between steps): the parameter
    after N steps of ``w -= lr * mean(x)`` equals the host computation."""
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import AllReduce
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=1), strategy_builder=AllReduce())
    with ad.scope():
        w = torch.nn.Parameter(torch.zeros(()))
        x = ad.placeholder((None, 1 << 18), torch.float32, name="x")
        loss = (w * x).mean()
        train_op = torch.optim.SGD([w], lr=1.0).minimize(loss)
        sess = ad.create_distributed_session()
        feeds = [torch.full((4, 1 << 18), float(i + 1)) for i in range(12)]
        for f in feeds:
            sess.run(train_op, {x: f})
        value = float(sess.run(w))
        sess.close()
    assert abs(value + sum(range(1, 13))) < 1e-3, value


@pytest.mark.parametrize("pinned", [True, False])
def test_prefetched_feed_is_used_by_the_next_step_and_gives_the_same_result(pinned):
    """``run(..., prefetch=next_feed)`` uploads the next batch while the step runs; feeding the same objects next must give
    what plain feeding gives, and a prefetched batch that is not fed next must simply be dropped."""
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.strategy import AllReduce
    results = []
    for use_prefetch in (False, True):
        _reset_default_autodist()
        ad = AutoDist(resource_spec=ResourceSpec.local(num_gpus=1), strategy_builder=AllReduce())
        with ad.scope():
            w = torch.nn.Parameter(torch.zeros(()))
            x = ad.placeholder((None, 1 << 16), torch.float32, name="x")
            loss = (w * x).mean()
            train_op = torch.optim.SGD([w], lr=1.0).minimize(loss)
            sess = ad.create_distributed_session()
            feeds = [torch.full((4, 1 << 16), float(i + 1)) for i in range(10)]
            if pinned:
                feeds = [f.pin_memory() for f in feeds]
            losses = []
            for i, f in enumerate(feeds):
                nxt = {x: feeds[i + 1]} if use_prefetch and i + 1 < len(feeds) else None
                if use_prefetch and i == 4:
                    nxt = {x: feeds[0]}                       # a prefetched batch that is never fed: dropped
                losses.append(float(sess.run([loss, train_op], {x: f}, prefetch=nxt)[0]))
            if use_prefetch:
                assert sess._remapper.h2d_bytes >= len(feeds) * feeds[0].numel() * 4
            results.append((losses, float(sess.run(w))))
            sess.close()
    assert results[0][1] == results[1][1] and results[0][0] == results[1][0], results
