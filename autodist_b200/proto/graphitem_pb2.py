"""``autodist.proto.GraphItem`` message (reference: ``autodist/proto/graphitem.proto:30-48``).

``graph_def`` carries the captured ``torch.fx`` graph (python code + tabular
node list wrapped in ``google.protobuf.Any`` holding a ``BytesValue``) in place
of a TensorFlow ``GraphDef``; ``Info.variables`` carry one serialized variable
record per parameter.
"""
from google.protobuf import any_pb2, wrappers_pb2  # noqa: F401  (register dependencies)

from autodist_b200.proto._build import declare_file

_classes = declare_file(
    "autodist_b200/proto/graphitem.proto", "autodist.proto",
    {
        "GraphItem": {
            "messages": {
                "Info": {"fields": [
                    ("variables", ".google.protobuf.Any", 1, {"repeated": True}),
                    ("table_initializers", "string", 2, {"repeated": True}),
                    ("savers", ".google.protobuf.Any", 3, {"repeated": True}),
                ]},
            },
            "fields": [
                ("graph_def", ".google.protobuf.Any", 1, {}),
                ("grad_target_pairs", "map<string,string>", 2, {}),
                ("info", ".autodist.proto.GraphItem.Info", 3, {}),
            ],
        },
    },
    dependencies=["google/protobuf/any.proto"])
GraphItem = _classes["GraphItem"]
