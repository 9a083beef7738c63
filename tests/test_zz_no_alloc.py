"""qt_matmul_f32_static: the allocation-free product for callers that cannot get device memory
at call time (fixed start-up arena, plain-C host without an allocator, latency-critical loop).
Its planes live in a 16 MiB array inside the library instead of caller-provided scratch.

Checked here through the C ABI: two calls in a row (the second reuses the array with the first
call's leftovers in it) against qt_matmul_f32 with caller scratch, and the size limit.
This file sorts last so that a run that stops at the first failure has run everything else."""
import ctypes as ct

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4          # relative Frobenius error, the tolerance of the other product tests


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def test_static_scratch_matches_caller_scratch_twice(native_lib):
    lib = native_lib
    dev = "cuda:0"
    P = lambda t: ct.c_void_p(t.data_ptr()) if t is not None else None
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=dev).manual_seed(23)
    # second case is smaller and transposed: it runs on top of the first call's leftovers
    cases = [(4, 384, 320, 512, False, False, 1.0, 0.0), (2, 200, 136, 96, True, True, -0.5, 2.0)]
    for b, M, N, K, ta, tb, alpha, beta in cases:
        A = torch.randn((b, K, M) if ta else (b, M, K), device=dev, generator=g)
        B = torch.randn((b, N, K) if tb else (b, K, N), device=dev, generator=g)
        C = torch.randn(b, M, N, device=dev, generator=g)
        want = torch.empty(b, M, N, device=dev)
        got = torch.full((b, M, N), float("nan"), device=dev)
        need = lib.qt_matmul_f32_scratch_bytes(M, N, K, b, int(ta), int(tb))
        assert need <= (16 << 20)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        rc = lib.qt_matmul_f32(P(A), A.stride(1), A.stride(0), int(ta), P(B), B.stride(1), B.stride(0), int(tb),
                               M, N, K, b, alpha, beta, P(C), N, M * N, P(want), N, M * N, P(scratch), need, st)
        assert rc == 0
        rc = lib.qt_matmul_f32_static(P(A), A.stride(1), A.stride(0), int(ta), P(B), B.stride(1), B.stride(0), int(tb),
                                      M, N, K, b, alpha, beta, P(C), N, M * N, P(got), N, M * N, st)
        assert rc == 0, lib.qt_error_string(rc)
        torch.cuda.synchronize()
        assert lib.qt_device_error(1) == 0
        assert torch.isfinite(got).all()
        assert torch.equal(got, want)                      # same kernels on the same planes: bit-identical
        ref = alpha * ((A.transpose(1, 2) if ta else A).double() @ (B.transpose(1, 2) if tb else B).double()) + beta * C.double()
        assert rel(got, ref) < TOL


def test_static_scratch_rejects_oversized_request(native_lib):
    lib = native_lib
    one = ct.c_void_p(256)
    # two 2048 x 2048 operands need 32 MiB of planes: refused before anything is touched or launched
    assert lib.qt_matmul_f32_scratch_bytes(2048, 2048, 2048, 1, 0, 0) > (16 << 20)
    rc = lib.qt_matmul_f32_static(one, 2048, 0, 0, one, 2048, 0, 0, 2048, 2048, 2048, 1, 1.0, 0.0,
                                  None, 0, 0, one, 2048, 0, None)
    assert rc == 8
    assert b"16 MiB" in lib.qt_error_string(rc)
    # sizes whose byte count would wrap around 2^64 are refused as well, not taken for small ones
    big = 1 << 30
    assert lib.qt_matmul_f32_scratch_bytes(big, big, big, 2, 0, 0) == 2 ** 64 - 1
    rc = lib.qt_matmul_f32_static(one, big, 0, 0, one, big, 0, 0, big, big, big, 2, 1.0, 0.0,
                                  None, 0, 0, one, big, 0, None)
    assert rc == 8
