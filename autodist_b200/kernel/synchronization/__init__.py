"""Gradient synchronizers: all-reduce (with compressors) and parameter-server."""
