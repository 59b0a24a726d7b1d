"""The allocation-free column-sum entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory where they call it (host callbacks, stream-ordered
regions owned by another library, fixed memory pools, latency-critical loops), so this one entry point keeps its
scratch inside the library. The test checks it against the ordinary entry point (which takes a scratch tensor from
the caller) on two calls in a row with different inputs, and that out-of-range requests are refused with a message.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from autodist_b200 import ops
    from autodist_b200.ops import build
    ops.ext(required=True)          # the shared object is loaded once; ctypes re-opens the same image
    lib = ctypes.CDLL(build.so_path())
    fn = lib.adb200_colsum_bf16_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.adb200_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def test_matches_the_allocating_entry_point_twice_in_a_row():
    from autodist_b200 import ops
    E = ops.ext(required=True)
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, cols) in enumerate([(4096, 1024), (300, 4096)]):
        torch.manual_seed(call)
        x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
        out = torch.full((cols,), float("nan"), device="cuda")
        rc = fn(x.data_ptr(), out.data_ptr(), rows, cols, stream)
        assert rc == 0, lib.adb200_noalloc_last_error()
        ref = torch.empty(cols, device="cuda")
        part = torch.empty(E.colsum_parts(rows) * cols, device="cuda")
        E.keyed_colsum(x, None, part, ref, 1, False)
        torch.cuda.synchronize()
        assert (out - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())
        plain = x.float().sum(0)
        assert (out - plain).abs().max().item() <= 1e-3 * max(1.0, plain.abs().max().item())


def test_refuses_what_the_scratch_cannot_hold():
    lib, fn = _lib()
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(8, device="cuda")
    assert fn(x.data_ptr(), out.data_ptr(), 8, 32768 + 8, None) == 10002
    assert b"exceeds" in lib.adb200_noalloc_last_error()
    assert fn(x.data_ptr(), out.data_ptr(), 8, 12, None) == 10001
    assert fn(None, out.data_ptr(), 8, 8, None) == 10003
    assert fn(x.data_ptr(), out.data_ptr(), 8, 8, None) == 0
    torch.cuda.synchronize()
    assert lib.adb200_noalloc_last_error() == b""
