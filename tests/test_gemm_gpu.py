"""tcgen05 bf16x3 matrix products (through the C ABI) against float64 torch.matmul.
Tolerance: 1e-4 relative Frobenius error (measured: ~1e-5)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4


def rel(a, b):
    return float((a.double() - b).norm() / b.norm())


def device_ok(lib):
    torch.cuda.synchronize()
    return lib.qt_device_error(1) == 0


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 128, 192), (100, 72, 50), (672, 672, 336), (1200, 1200, 768)])
def test_matmul_all_majors(native_lib, trans_a, trans_b, M, N, K):
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    b = 2
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    D, _ = _gemm.matmul(_gemm.split(A), _gemm.split(B), trans_a=trans_a, trans_b=trans_b)
    assert device_ok(native_lib)
    ref = (A.transpose(1, 2) if trans_a else A).double() @ (B.transpose(1, 2) if trans_b else B).double()
    assert rel(D, ref) < TOL, rel(D, ref)


def test_alpha_beta_c_and_plane_output(native_lib):
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(5)
    b, M, N, K = 3, 200, 328, 136
    A = torch.randn(b, M, K, device="cuda", generator=g)
    B = torch.randn(b, K, N, device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D, P = _gemm.matmul(_gemm.split(A), _gemm.split(B), alpha=-0.5, beta=1.5, C=C, want_planes=True)
    assert device_ok(native_lib)
    ref = -0.5 * (A.double() @ B.double()) + 1.5 * C.double()
    assert rel(D, ref) < TOL
    assert rel(P.to_float(), ref) < TOL
    # output canary: a padded output buffer keeps its guard columns
    big = torch.full((b, M, N + 8), 7.0, device="cuda")
    _gemm.matmul(_gemm.split(A), _gemm.split(B), out=big[:, :, :N])
    assert device_ok(native_lib)
    assert bool((big[:, :, N:] == 7.0).all())
    assert rel(big[:, :, :N], A.double() @ B.double()) < TOL


def test_split_planes_are_exact_to_16_bits(native_lib):
    from optimizers import _gemm
    X = torch.randn(2, 77, 130, device="cuda") * torch.logspace(-3, 3, 130, device="cuda")
    P = _gemm.split(X)
    err = (P.to_float() - X).abs() / X.abs().clamp_min(1e-30)
    assert float(err.max()) < 2.0 ** -15


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True)])
def test_matmul_f32_entry_point_with_caller_scratch(native_lib, trans_a, trans_b):
    """qt_matmul_f32: fp32 operands, planes built in caller-provided scratch memory."""
    import ctypes as ct
    lib = native_lib
    g = torch.Generator(device="cuda").manual_seed(17)
    b, M, N, K = 3, 320, 200, 456
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D = torch.empty(b, M, N, device="cuda")
    need = lib.qt_matmul_f32_scratch_bytes(M, N, K, b, int(trans_a), int(trans_b))
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    P = lambda t: ct.c_void_p(t.data_ptr())
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.qt_matmul_f32(P(A), A.stride(1), A.stride(0), int(trans_a), P(B), B.stride(1), B.stride(0), int(trans_b),
                           M, N, K, b, 2.0, -1.0, P(C), N, M * N, P(D), N, M * N, P(scratch), need, st)
    assert rc == 0 and device_ok(lib)
    ref = 2.0 * ((A.transpose(1, 2) if trans_a else A).double() @ (B.transpose(1, 2) if trans_b else B).double()) - C.double()
    assert rel(D, ref) < TOL
    # too little scratch is refused before anything is launched
    assert lib.qt_matmul_f32(P(A), A.stride(1), A.stride(0), int(trans_a), P(B), B.stride(1), B.stride(0), int(trans_b),
                             M, N, K, b, 1.0, 0.0, None, 0, 0, P(D), N, M * N, P(scratch), need - 4096, st) == 1


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (True, False), (False, False)])
def test_three_plane_product_reaches_fp32_accuracy(native_lib, trans_a, trans_b):
    """hi/mid/lo planes, six MMAs per k-slice: at least as accurate as an fp32 library product."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(31)
    b, M, N, K = 2, 328, 264, 1200
    A = torch.randn((b, K, M) if trans_a else (b, M, K), device="cuda", generator=g)
    B = torch.randn((b, N, K) if trans_b else (b, K, N), device="cuda", generator=g)
    C = torch.randn(b, M, N, device="cuda", generator=g)
    D, _ = _gemm.matmul(_gemm.split3(A), _gemm.split3(B), trans_a=trans_a, trans_b=trans_b, alpha=0.05, beta=0.95, C=C)
    assert device_ok(native_lib)
    opA = A.transpose(1, 2) if trans_a else A
    opB = B.transpose(1, 2) if trans_b else B
    ref = 0.05 * (opA.double() @ opB.double()) + 0.95 * C.double()
    fp32 = torch.baddbmm(C, opA, opB, beta=0.95, alpha=0.05)
    assert rel(D, ref) < 2e-6, rel(D, ref)               # measured 8e-7, independent of K
    assert rel(D, ref) < 4 * rel(fp32, ref) + 1e-6
    P = _gemm.split3(A)
    back = P.hi.float() + P.mid.float() + P.lo.float()
    assert float((back.view(-1)[: A.numel()].view_as(A) - A).abs().max() / A.abs().max()) < 2.0 ** -22
