"""``autodist.proto.PSSynchronizer`` / ``AllReduceSynchronizer`` messages.

Field numbers follow the reference's ``autodist/proto/synchronizers.proto:25-57``.
Two additions: compressor value ``PowerSGDCompressor = 3`` (commented out at
``synchronizers.proto:50`` in the reference) and ``power_sgd_rank = 4``.
"""
from autodist_b200.proto._build import declare_file

_classes = declare_file(
    "autodist_b200/proto/synchronizers.proto", "autodist.proto",
    {
        "PSSynchronizer": {"fields": [
            ("reduction_destination", "string", 1, {}),
            ("local_replication", "bool", 2, {}),
            ("sync", "bool", 3, {}),
            ("staleness", "int32", 4, {}),
        ]},
        "AllReduceSynchronizer": {
            "enums": {
                "Spec": [("AUTO", 0), ("NCCL", 1), ("RING", 2)],
                "Compressor": [("NoneCompressor", 0), ("HorovodCompressor", 1), ("HorovodCompressorEF", 2),
                               ("PowerSGDCompressor", 3)],
            },
            "fields": [
                ("spec", ".autodist.proto.AllReduceSynchronizer.Spec", 1, {"enum": True}),
                ("compressor", ".autodist.proto.AllReduceSynchronizer.Compressor", 2, {"enum": True}),
                ("group", "int32", 3, {}),
                ("power_sgd_rank", "int32", 4, {}),
            ],
        },
    })
PSSynchronizer = _classes["PSSynchronizer"]
AllReduceSynchronizer = _classes["AllReduceSynchronizer"]
