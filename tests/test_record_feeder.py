"""The native background batch feeder (``csrc/host/batch_feeder.cpp``) behind ``utils.data.RecordFeeder``."""
import numpy as np
import pytest
import torch

from autodist_b200.utils.data import RecordFeeder, read_fields, write_records


@pytest.fixture()
def record_file(tmp_path):
    n = 103
    x = torch.arange(n, dtype=torch.float32)[:, None] * torch.ones(1, 4)          # row i holds i in every element
    y = torch.arange(n, dtype=torch.int64) * 10
    m = (torch.arange(n) % 2 == 0)
    path = str(tmp_path / "samples.rec")
    fields = write_records(path, {"x": x, "y": y, "m": m})
    assert fields == {"x": ((4,), torch.float32), "y": ((), torch.int64), "m": ((), torch.bool)}
    assert read_fields(path) == fields
    return path, n


def _ids(batch):
    assert torch.equal(batch["x"], batch["x"][:, :1].expand(-1, 4)) and torch.equal(batch["y"], (batch["x"][:, 0] * 10).long())
    assert torch.equal(batch["m"], batch["y"] % 20 == 0)
    return batch["x"][:, 0].long().tolist()


def test_sequential_order_and_short_last_batch(record_file):
    path, n = record_file
    feeder = RecordFeeder(path, 10, shuffle=False, drop_last=False, depth=2, workers=4)
    seen = [_ids(b) for b in feeder]
    assert [len(s) for s in seen] == [10] * 10 + [3]
    assert sum(seen, []) == list(range(n))
    assert feeder.batches_per_epoch == 11 and feeder.records == n
    feeder.close()


def test_shuffle_is_seeded_differs_between_epochs_and_covers_every_record(record_file):
    path, n = record_file
    a = [_ids(b) for b in RecordFeeder(path, 10, shuffle=True, seed=5, drop_last=False, epochs=2, workers=3, depth=4)]
    b = [_ids(b) for b in RecordFeeder(path, 10, shuffle=True, seed=5, drop_last=False, epochs=2, workers=1, depth=2)]
    c = [_ids(b) for b in RecordFeeder(path, 10, shuffle=True, seed=6, drop_last=False, epochs=1)]
    assert a == b                                                     # the order does not depend on threads or ring depth
    first, second = sum(a[:11], []), sum(a[11:], [])
    assert sorted(first) == list(range(n)) and sorted(second) == list(range(n)) and first != second
    assert sum(c, []) != first and first != list(range(n))


def test_replicas_draw_disjoint_equal_parts_of_one_permutation(record_file):
    path, n = record_file
    parts = []
    for rank in range(4):
        batches = [_ids(b) for b in RecordFeeder(path, 5, shuffle=True, seed=1, drop_last=True, rank=rank, world=4)]
        assert [len(s) for s in batches] == [5] * 5                    # 103 // 4 = 25 records per rank
        parts.append(sum(batches, []))
    flat = sum(parts, [])
    assert len(set(flat)) == len(flat) == 100


def test_a_batch_stays_valid_while_the_next_one_is_drawn(record_file):
    """The loop shape of ``run(feed=batch_i, prefetch=batch_{i+1})``: batch i is still read after batch i + 1 was drawn."""
    path, n = record_file
    feeder = RecordFeeder(path, 7, shuffle=False, drop_last=True, depth=3, workers=2, epochs=3)
    it = iter(feeder)
    current = next(it)
    count, expect = 0, 0
    for nxt in it:
        ids = _ids(current)                                            # read after the following batch exists
        assert ids == [(expect + j) % (14 * 7) for j in range(7)]
        expect = (expect + 7) % (14 * 7)
        current = nxt
        count += 1
    assert count == 3 * 14 - 1


def test_bad_arguments_are_refused(record_file, tmp_path):
    path, n = record_file
    with pytest.raises(ValueError):
        RecordFeeder(path, 10, depth=1)
    with pytest.raises(RuntimeError):
        RecordFeeder(path, 200)                                        # fewer records than one batch
    with pytest.raises(RuntimeError):
        RecordFeeder(str(tmp_path / "missing.rec"), 4, fields={"x": ((4,), torch.float32)})
    with pytest.raises(ValueError):
        write_records(str(tmp_path / "bad.rec"), {"a": np.zeros((3, 2)), "b": np.zeros((4,))})
