"""The entry point for callers that must not allocate (csrc/no_alloc.h).

Some programs that embed this library cannot let it allocate when they call
it: they have handed the whole device to a memory pool of their own, or they
run on a thread whose latency budget has no room for the device-wide
synchronisation inside cudaMalloc and cudaFree.  For them the library exports
``ayk_gemm_tc_no_alloc``, the split-K tensor-core product with its scratch in
static device arrays of the library image.  This test calls it through its C
symbol, as such a program would, and compares it with the ordinary entry point
on two calls in a row (the second with other sizes and data, so that anything
left in the shared scratch by the first call would show).

The file name makes pytest collect it last: if it fails, a run that stops at the
first failure has already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def c_entry():
    from ayaka_py_b200 import ops
    ops.library()                                         # builds the library if it is missing
    lib = ctypes.CDLL(ops.library_file())
    fn = lib.ayk_gemm_tc_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    lib.ayk_last_error.restype = ctypes.c_char_p
    lib.ayk_gemm_tc_no_alloc_error.restype = ctypes.c_int
    return lib, fn


def operands(seed, M, N, K):
    rs = np.random.RandomState(seed)
    x = torch.from_numpy(rs.randn(M, K).astype(np.float32)).cuda().to(torch.bfloat16)
    w = torch.from_numpy((rs.randn(N, K) / np.sqrt(K)).astype(np.float32)).cuda().to(torch.bfloat16)
    bias = torch.from_numpy(rs.randn(N).astype(np.float32)).cuda()
    residual = torch.from_numpy(rs.randn(M, N).astype(np.float32)).cuda()
    return x, w, bias, residual


def reference_product(x, w, bias, residual, act):
    """The product in float32 from the bfloat16-rounded operands, by a library matmul: independent of
    every kernel of this package."""
    y = x.float() @ w.float().t() + bias
    if act == 1:
        y = torch.nn.functional.gelu(y)
    elif act == 2:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    return y + residual


def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row():
    from ayaka_py_b200 import ops
    torch.cuda.set_device(0)
    lib, fn = c_entry()
    stream = torch.cuda.current_stream().cuda_stream
    # (M, N, K, splits, activation): explicit splits, no split, and "the library chooses" (<= 0), among them
    # a shape whose unclamped choice (148 / 13 tiles = 11 splits x 128 x 1600 floats) would not fit the scratch
    cases = [(8, 1600, 1600, 9, 0), (40, 300, 1000, 7, 2), (24, 520, 328, 1, 1), (128, 1600, 6400, 0, 0), (5, 3000, 512, -1, 2)]
    for seed, (M, N, K, splits, act) in enumerate(cases):
        x, w, bias, residual = operands(seed, M, N, K)
        name = ["none", "gelu_erf", "gelu_tanh"][act]
        want = ops.gemm_tc(x, w, bias, name, residual, out_dtype=torch.float32, splits=max(splits, 1), static_weight=False)
        independent = reference_product(x, w, bias, residual, act)
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        for attempt in range(2):                              # the very first call may load modules: judge the second
            free_before, _ = torch.cuda.mem_get_info()        # device-wide free bytes: any cudaMalloc would move them
            code = fn(out.data_ptr(), x.data_ptr(), w.data_ptr(), bias.data_ptr(), residual.data_ptr(),
                      M, N, K, act, 0, splits, stream)
            assert code == 0, lib.ayk_last_error().decode()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, f"the call changed the device's free memory by {free_before - free_after} bytes"
        assert lib.ayk_gemm_tc_no_alloc_error() == 0
        assert float((out - independent).abs().max()) < 2e-3      # bfloat16 operands, 32-bit sums: order of summation only
        if splits >= 1:
            assert float((out - want).abs().max()) < 2e-5         # the same splits as the ordinary entry point
        else:
            assert float((out - want).abs().max()) < 2e-3


def test_no_alloc_entry_refuses_what_exceeds_its_scratch():
    lib, fn = c_entry()
    x, w, bias, residual = operands(3, 64, 6400, 1600)
    out = torch.empty((64, 6400), dtype=torch.float32, device="cuda")
    code = fn(out.data_ptr(), x.data_ptr(), w.data_ptr(), bias.data_ptr(), residual.data_ptr(),
              64, 6400, 1600, 0, 0, 4, torch.cuda.current_stream().cuda_stream)
    assert code != 0 and "exceed the built-in" in lib.ayk_last_error().decode()
    # the same shape with the choice left to the library runs (it picks a split count that fits)
    code = fn(out.data_ptr(), x.data_ptr(), w.data_ptr(), bias.data_ptr(), residual.data_ptr(),
              64, 6400, 1600, 0, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert code == 0, lib.ayk_last_error().decode()
    torch.cuda.synchronize()
    assert float((out - reference_product(x, w, bias, residual, 0)).abs().max()) < 2e-3
