"""Protobuf messages of the strategy representation.

The message and field numbers are wire-compatible with the reference's
``autodist/proto/{synchronizers,strategy,graphitem}.proto``; the descriptors
are built in Python (see ``_build.py``) because the toolchain has no ``protoc``.
"""
from autodist_b200.proto import graphitem_pb2, strategy_pb2, synchronizers_pb2  # noqa: F401
