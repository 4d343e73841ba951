"""The entry point that allocates nothing, called through its exported C symbol.

``bw_bf16_linear_noalloc`` serves callers that must not allocate device memory when they need
a matrix product (code inside a stream capture, inside another framework's memory pool, in
a latency-critical loop, or with a fixed memory budget): they hand in inputs and outputs they
already own, and the scratch of the split summation lives in a fixed array inside the
library.  It must give the bits of the ordinary entry point, on two calls in a row (the
scratch keeps the first call's contents), for products that use the scratch and for products
that do not, and it must refuse a product whose scratch would not fit.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib_and_ops():
    from bitwise_b200.kernels.ops import get_ops
    ops = get_ops("bfloat16")
    lib = ctypes.CDLL(ops.library_path)  # the same shared library, opened by its path
    fn = lib.bw_bf16_linear_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.bw_last_error.restype = ctypes.c_char_p
    return lib, fn, ops


def _call(fn, x, w, y, residual, stream):
    m, k = x.shape
    n = w.shape[0]
    return fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), int(y.dtype == torch.float32),
              residual.data_ptr() if residual is not None else None, m, n, k, stream)


@pytest.mark.parametrize("m,n,k,uses_scratch", [(8, 2048, 8192, True), (64, 1024, 4096, True), (1, 2304, 6152, True),
                                                (8, 16384, 2048, True), (200, 384, 1024, False),
                                                (8, 49152, 2048, False), (100, 16384, 2048, False),
                                                (16, 512, 512, False)])
def test_no_alloc_entry_gives_the_bits_of_the_ordinary_one_twice_in_a_row(m, n, k, uses_scratch):
    lib, fn, ops = _lib_and_ops()
    assert bool(lib.bw_bf16_linear_tc_splits(m, n, k)) == uses_scratch
    # what the header promises about the scratch: chunks of 512 along k, times m, times n
    lib.bw_bf16_linear_noalloc_scratch_floats.restype = ctypes.c_longlong
    assert lib.bw_bf16_linear_noalloc_scratch_floats(m, n, k) == (((k + 511) // 512) * m * n if uses_scratch else 0)
    g = torch.Generator(device="cuda:0").manual_seed(m + n + k)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):  # the second call finds the first call's chunk sums in the scratch
        x = torch.randn(m, k, device="cuda:0", generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda:0", generator=g) * 0.05).to(torch.bfloat16)
        res = torch.randn(m, n, device="cuda:0", generator=g)
        want32 = res.clone()
        ops.linear(x, w, want32, residual=want32)
        want16 = torch.empty(m, n, device="cuda:0", dtype=torch.bfloat16)
        ops.linear(x, w, want16)
        got32 = res.clone()
        rc = _call(fn, x, w, got32, got32, stream)
        assert rc == 0, lib.bw_last_error().decode()
        got16 = torch.empty_like(want16)
        rc = _call(fn, x, w, got16, None, stream)
        assert rc == 0, lib.bw_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(got32.view(torch.int32), want32.view(torch.int32)), f"call {call}: float32 output differs"
        assert torch.equal(got16.view(torch.int16), want16.view(torch.int16)), f"call {call}: bfloat16 output differs"
        ref = res.double() + x.double() @ w.double().t()
        assert float((got32.double() - ref).abs().max()) <= 1e-4 * float(ref.abs().max())
    assert not ops.device_failure() and not lib.bw_bf16_linear_noalloc_failed()


def test_no_alloc_entry_refuses_what_does_not_fit():
    lib, fn, ops = _lib_and_ops()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    m, n, k = 16, 8192, 32768  # 64 chunks * 16 * 8192 floats = 8.4 M > 4 M
    x = torch.zeros(m, k, device="cuda:0", dtype=torch.bfloat16)
    w = torch.zeros(n, k, device="cuda:0", dtype=torch.bfloat16)
    y = torch.zeros(m, n, device="cuda:0")
    assert lib.bw_bf16_linear_tc_splits(m, n, k)
    rc = _call(fn, x, w, y, None, stream)
    assert rc < 0 and b"scratch" in lib.bw_last_error()
    # rows that do not start on 16 bytes are refused too, with a reason
    x2 = torch.zeros(4, 100, device="cuda:0", dtype=torch.bfloat16)
    w2 = torch.zeros(16, 100, device="cuda:0", dtype=torch.bfloat16)
    y2 = torch.zeros(4, 16, device="cuda:0")
    rc = _call(fn, x2, w2, y2, None, stream)
    assert rc < 0 and b"16 bytes" in lib.bw_last_error()
