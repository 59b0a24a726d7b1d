"""Strategy wrapper: ids, serialisation, wire compatibility with the reference's field numbers."""
import os

from autodist_b200.proto import strategy_pb2, synchronizers_pb2
from autodist_b200.strategy.base import Strategy


def test_id_and_round_trip(tmp_path):
    s = Strategy()
    assert len(s.id) >= 20 and "T" in s.id and "M" in s.id
    n = s.node_config.add(var_name="w:0")
    n.PSSynchronizer.reduction_destination = "localhost:CPU:0"
    n.PSSynchronizer.sync = True
    s.graph_config.replicas.extend(["localhost:GPU:0", "localhost:GPU:1"])
    path = s.serialize(str(tmp_path / s.id))
    assert os.path.exists(path) and s.path == path
    assert Strategy.deserialize(path=path) == s
    s.serialize()
    assert Strategy.deserialize(s.id) == s


def test_wire_format_matches_reference_field_numbers():
    """Bytes hand-assembled from the reference's .proto field numbers parse into the same message."""
    # Strategy{ id(1)="x", node_config(3){ var_name(1)="w:0", AllReduceSynchronizer(3){spec(1)=1, compressor(2)=2, group(3)=5},
    #           partitioner(4)="2,1" }, graph_config(4){ replicas(1)="a" } }
    ar = bytes([0x08, 1, 0x10, 2, 0x18, 5])
    node = bytes([0x0A, 3]) + b"w:0" + bytes([0x1A, len(ar)]) + ar + bytes([0x22, 3]) + b"2,1"
    gc = bytes([0x0A, 1]) + b"a"
    raw = bytes([0x0A, 1]) + b"x" + bytes([0x1A, len(node)]) + node + bytes([0x22, len(gc)]) + gc
    msg = strategy_pb2.Strategy.FromString(raw)
    assert msg.id == "x" and msg.graph_config.replicas == ["a"]
    n = msg.node_config[0]
    assert n.var_name == "w:0" and n.partitioner == "2,1"
    assert n.WhichOneof("synchronizer") == "AllReduceSynchronizer"
    assert n.AllReduceSynchronizer.spec == synchronizers_pb2.AllReduceSynchronizer.NCCL
    assert n.AllReduceSynchronizer.compressor == synchronizers_pb2.AllReduceSynchronizer.HorovodCompressorEF
    assert n.AllReduceSynchronizer.group == 5
    assert msg.SerializeToString() == raw


def test_ps_fields():
    ps = synchronizers_pb2.PSSynchronizer(reduction_destination="h:CPU:0", local_replication=True, sync=True, staleness=3)
    raw = ps.SerializeToString()
    assert raw == bytes([0x0A, 7]) + b"h:CPU:0" + bytes([0x10, 1, 0x18, 1, 0x20, 3])
