"""The symmetric-memory barrier protocol, run as host threads (one per rank and block) by the C++ model."""
import pytest

from autodist_b200.ops import build


@pytest.fixture(scope="module")
def model():
    return build.load_host()


@pytest.mark.parametrize("world,blocks,n", [(1, 1, 5), (2, 1, 1), (2, 4, 257), (3, 5, 1009), (4, 3, 64), (8, 2, 4099)])
def test_packed_two_shot_all_reduce_is_exact(model, world, blocks, n):
    errors, max_err = model.simulate_allreduce(world, blocks, n, iters=4, timeout_ms=20000.0)
    assert errors == [0] * world
    assert max_err <= 1e-4


def test_epochs_survive_wrap_around(model):
    # flags start three steps before 2**32; two barriers per all-reduce carry them across the wrap
    errors, max_err = model.simulate_allreduce(2, 4, 513, iters=6, first_epoch=0xFFFFFFFD, timeout_ms=20000.0)
    assert errors == [0, 0] and max_err <= 1e-4


def test_absent_rank_is_reported_not_waited_for(model):
    errors, _ = model.simulate_allreduce(4, 3, 1001, iters=2, absent=[2], timeout_ms=1500.0)
    assert errors[2] == 0                           # it never ran
    assert all(e == 102 for i, e in enumerate(errors) if i != 2)     # 100 + the peer that never arrived


def test_size_checks(model):
    with pytest.raises(ValueError):
        model.simulate_allreduce(0, 1, 8)
    with pytest.raises(ValueError):
        model.simulate_allreduce(2, 65, 8)


@pytest.mark.parametrize("staleness", [0, 1, 3])
def test_staleness_gate_bounds_the_lead_of_the_fast_rank(model, staleness):
    # rank 1 is slow (2 ms of work per step); nothing here asserts on elapsed time, only on how far ahead anyone got
    lead, errors, reached = model.simulate_staleness(3, 12, staleness, delays_us=[0, 2000, 0], timeout_ms=20000.0)
    assert errors == [0, 0, 0] and reached == [12, 12, 12]
    assert max(lead) <= staleness
    if staleness:
        assert max(lead[0], lead[2]) >= 1                          # the fast ranks do use slack they are given


def test_staleness_gate_reports_a_rank_that_stopped(model):
    # rank 2 stops publishing after step 2 (a process that left between steps): the others get staleness steps further
    lead, errors, reached = model.simulate_staleness(3, 10, 1, timeout_ms=1500.0, stop_after=[10, 10, 2])
    assert errors[2] == 0 and reached[2] == 2
    assert errors[0] == 202 and errors[1] == 202
    assert reached[0] == 3 and reached[1] == 3                      # step 4 would be 2 ahead of rank 2
