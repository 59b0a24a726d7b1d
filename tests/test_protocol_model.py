"""The symmetric-memory barrier protocol, run as host threads (one per rank and block) by the C++ model."""
import pytest

from autodist_b200.ops import build


@pytest.fixture(scope="module")
def model():
    return build.load_host()


@pytest.mark.parametrize("world,blocks,n", [(1, 1, 5), (2, 1, 1), (2, 4, 257), (3, 5, 1009), (4, 3, 64), (8, 2, 4099)])
def test_packed_two_shot_all_reduce_is_exact(model, world, blocks, n):
    errors, max_err = model.simulate_allreduce(world, blocks, n, iters=4)
    assert errors == [0] * world
    assert max_err <= 1e-4


def test_epochs_survive_wrap_around(model):
    # flags start three steps before 2**32; two barriers per all-reduce carry them across the wrap
    errors, max_err = model.simulate_allreduce(2, 4, 513, iters=6, first_epoch=0xFFFFFFFD)
    assert errors == [0, 0] and max_err <= 1e-4


def test_absent_rank_is_reported_not_waited_for(model):
    errors, _ = model.simulate_allreduce(4, 3, 1001, iters=2, absent=[2], timeout_ms=100.0)
    assert errors[2] == 0                           # it never ran
    assert all(e == 102 for i, e in enumerate(errors) if i != 2)     # 100 + the peer that never arrived


def test_size_checks(model):
    with pytest.raises(ValueError):
        model.simulate_allreduce(0, 1, 8)
    with pytest.raises(ValueError):
        model.simulate_allreduce(2, 65, 8)
