"""The entry point for callers that cannot allocate: li_gemm_skinny_static (csrc/gemm_skinny_static.h).

Some hosts of the kernel library may not call cudaMalloc at all (a plug-in inside someone else's CUDA
context, a loop that must stay clear of the driver's allocator, a sandbox that forbids it).  For them
the k-sliced decode product keeps its partial sums in a fixed array inside the library.  This test calls
that function through its exported C symbol, the way such a host would, and compares it with the
ordinary entry point, which takes its scratch from the caller.

Collected last on purpose: if it fails, a run that stops at the first failure has run everything else.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_size_t, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_SMALL = 100003


def _library():
    from liteinfer_b200.ops.library import load

    lib = load("gemm_skinny_static")
    lib.li_gemm_skinny_static.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.li_gemm_skinny_static.restype = c_int
    lib.li_gemm_skinny_static_needs.argtypes = [c_int, c_int, c_int]
    lib.li_gemm_skinny_static_needs.restype = c_size_t
    lib.li_static_error_string.argtypes = [c_int]
    lib.li_static_error_string.restype = ctypes.c_char_p
    return lib


def _inputs(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g, device="cuda").to(torch.bfloat16)
    return x, w, b


def test_static_scratch_product_matches_the_ordinary_one_twice_in_a_row():
    from liteinfer_b200 import ops

    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    # The first call on a device looks up the array's address; do it before anything is measured.
    x, w, b = _inputs(2, 2048, 8192, 0)
    out = torch.empty(2, 2048, dtype=torch.bfloat16, device="cuda")
    assert lib.li_gemm_skinny_static(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 2, 2048, 8192, stream) == 0
    torch.cuda.synchronize()

    cases = [(8, 2048, 8192, 1), (3, 3072, 2048, 2)]       # both sliced over k, so both use the array
    prepared = []
    for M, N, K, seed in cases:
        assert lib.li_gemm_skinny_static_needs(M, N, K) > 0
        x, w, b = _inputs(M, N, K, seed)
        prepared.append((x, w, b, torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda"),
                         ops.gemm_skinny(x, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"), b)))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for (M, N, K, _), (x, w, b, out, _) in zip(cases, prepared):    # two calls in a row, nothing in between
        code = lib.li_gemm_skinny_static(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, stream)
        assert code == 0, lib.li_static_error_string(code).decode()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before                        # nothing was allocated along the way
    for x, w, b, out, want in prepared:
        torch.testing.assert_close(out.float(), want.float(), rtol=2 ** -7, atol=2 ** -7)
        exact = x.double() @ w.double().t() + b.double()
        torch.testing.assert_close(out.double(), exact, rtol=2 ** -7, atol=2 ** -7)


def test_static_scratch_refuses_what_does_not_fit():
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    M, N, K = 64, 2048, 8192                                # 64 rows of x, eight slices of k: 1 Mi floats
    assert lib.li_gemm_skinny_static_needs(M, N, K) > (1 << 18)
    x, w, _ = _inputs(M, N, K, 3)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    code = lib.li_gemm_skinny_static(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, K, stream)
    assert code == TOO_SMALL and b"scratch" in lib.li_static_error_string(code)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0                    # nothing was launched
    assert lib.li_gemm_skinny_static(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 65, N, K, stream) == 100001
    # A shape that is not sliced needs no scratch at all and always runs.
    assert lib.li_gemm_skinny_static_needs(64, 16384, 2048) == 0
