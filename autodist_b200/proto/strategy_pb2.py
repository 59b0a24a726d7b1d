"""``autodist.proto.Strategy`` message (reference: ``autodist/proto/strategy.proto:30-69``)."""
from autodist_b200.proto import synchronizers_pb2  # noqa: F401  (registers the dependency first)
from autodist_b200.proto._build import declare_file

_classes = declare_file(
    "autodist_b200/proto/strategy.proto", "autodist.proto",
    {
        "Strategy": {
            "messages": {
                "Node": {
                    "oneofs": ["synchronizer"],
                    "fields": [
                        ("var_name", "string", 1, {}),
                        ("PSSynchronizer", ".autodist.proto.PSSynchronizer", 2, {"oneof": "synchronizer"}),
                        ("AllReduceSynchronizer", ".autodist.proto.AllReduceSynchronizer", 3,
                         {"oneof": "synchronizer"}),
                        ("partitioner", "string", 4, {}),
                        ("part_config", ".autodist.proto.Strategy.Node", 5, {"repeated": True}),
                    ],
                },
                "GraphConfig": {"fields": [("replicas", "string", 1, {"repeated": True})]},
            },
            "fields": [
                ("id", "string", 1, {}),
                ("path", "string", 2, {}),
                ("node_config", ".autodist.proto.Strategy.Node", 3, {"repeated": True}),
                ("graph_config", ".autodist.proto.Strategy.GraphConfig", 4, {}),
            ],
        },
    },
    dependencies=["autodist_b200/proto/synchronizers.proto"])
Strategy = _classes["Strategy"]
