"""Schur-Newton inverse root inside the library (qt_power_iter, qt_inverse_root_newton, the
extras of qt_gemm_ex) against the CPU oracle's statement of the reference algorithm
(optimizers/matrix_functions.py:22-141).  Tolerance: 1e-4 relative Frobenius error where the
input is well conditioned; for the 1e6-conditioned spectrum of the kernel-sweep configuration
the comparison is against the exact inverse root in float64, where the library must be as close
as the fp32 oracle is (any fp32 evaluation is off by ~ eps * cond / 4 there)."""
import ctypes as ct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def spd(n, lo, seed):
    """Q diag(lambda) Q^T with lambda log-uniform in [lo, 1] (float64 construction, fp32 result)."""
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g))
    lam = torch.exp(torch.empty(n, dtype=torch.float64).uniform_(float(np.log(lo)), 0.0, generator=g))
    a = (q * lam) @ q.T
    return (0.5 * (a + a.T)).float()


@pytest.mark.parametrize("n", [64, 100, 768])
def test_power_iteration_follows_the_reference_step_by_step(native_lib, n):
    from optimizers import matrix_functions as MF
    from oracle.shampoo_oracle import power_iter
    mats = [spd(n, 1e-3, 10 + k) for k in range(3)]
    g = torch.Generator().manual_seed(1)
    v0 = torch.rand(3, n, generator=g) * 2 - 1
    sval, vec, iters = MF.PowerIter(torch.stack(mats).cuda(), v0=v0.cuda())
    torch.cuda.synchronize()
    for k in range(3):
        want = power_iter(mats[k], v0=v0[k])
        assert abs(float(sval[k]) - float(want)) <= 2e-6 * float(want)
        assert 1 <= int(iters[k]) <= 10
        assert abs(float(vec[k].norm()) - 1.0) < 1e-5


@pytest.mark.parametrize("n", [64, 100, 336, 768, 1200])
def test_inverse_root_matches_oracle_on_well_conditioned_input(native_lib, n):
    from optimizers import matrix_functions as MF
    from oracle.shampoo_oracle import newton_inverse_root
    mats = [spd(n, 1e-2, 100 + n + k) for k in range(3)]
    g = torch.Generator().manual_seed(2)
    v0 = torch.rand(3, n, generator=g) * 2 - 1
    G = torch.stack(mats).cuda()
    keep = G.clone()
    root = MF.ComputePower(G, 4, ridge_epsilon=1e-6, v0=v0.cuda())
    torch.cuda.synchronize()
    assert native_lib.qt_device_error(1) == 0
    # the ridge was added in place, as in the reference (matrix_functions.py:112)
    delta = G - keep
    assert float(delta.diagonal(dim1=1, dim2=2).min()) > 0
    assert float((delta - torch.diag_embed(delta.diagonal(dim1=1, dim2=2))).abs().max()) == 0.0
    for k in range(3):
        want = newton_inverse_root(mats[k].clone(), 4, ridge=1e-6, v0=v0[k])
        e = rel(root[k].cpu(), want)
        print(f"order {n} matrix {k}: inverse root error vs oracle {e:.3e}")
        assert e < TOL, (n, k, e)


@pytest.mark.parametrize("n", [128, 512, 1200])
def test_inverse_root_on_sweep_spectrum_is_as_accurate_as_fp32_allows(native_lib, n):
    """Spectrum log-uniform in [1e-6, 1] (the kernel-sweep configuration): both the library and
    the fp32 oracle are compared with the exact (float64, eigendecomposition) inverse root."""
    from optimizers import matrix_functions as MF
    from oracle.shampoo_oracle import newton_inverse_root, power_iter
    A = spd(n, 1e-6, 7 + n)
    g = torch.Generator().manual_seed(3)
    v0 = torch.rand(n, generator=g) * 2 - 1
    root = MF.ComputePower(A.clone().cuda().unsqueeze(0), 4, ridge_epsilon=1e-6, v0=v0.cuda().unsqueeze(0))[0].cpu()
    want32 = newton_inverse_root(A.clone(), 4, ridge=1e-6, v0=v0)
    ridge = 1e-6 * float(power_iter(A, v0=v0))
    w, Q = torch.linalg.eigh(A.double() + ridge * torch.eye(n, dtype=torch.float64))
    exact = (Q * w.clamp_min(1e-300).pow(-0.25)) @ Q.T
    e_lib, e_ora = rel(root, exact), rel(want32, exact)
    print(f"order {n}: library {e_lib:.3e}, fp32 oracle {e_ora:.3e} (vs exact)")
    assert torch.isfinite(root).all()
    assert e_lib < max(TOL, 3 * e_ora), (n, e_lib, e_ora)


def test_per_matrix_stop_rule_and_single_matrix_form(native_lib):
    """A batch in which one matrix is already converged (identity scaled so that M = I), one
    is well conditioned and one is ill conditioned: each follows its own stop rule; the 2-D
    (single matrix) call gives the same bytes as the batched one."""
    from optimizers import matrix_functions as MF
    from oracle.shampoo_oracle import newton_inverse_root
    n = 192
    mats = [torch.eye(n) * 2.5, spd(n, 1e-1, 5), spd(n, 1e-5, 6)]
    g = torch.Generator().manual_seed(4)
    v0 = torch.rand(3, n, generator=g) * 2 - 1
    root = MF.ComputePower(torch.stack(mats).cuda(), 4, v0=v0.cuda())
    single = MF.ComputePower(mats[1].clone().cuda(), 4, v0=v0[1].cuda())
    torch.cuda.synchronize()
    assert torch.equal(single, root[1])
    for k in range(2):
        want = newton_inverse_root(mats[k].clone(), 4, v0=v0[k])
        assert rel(root[k].cpu(), want) < TOL, k
    assert torch.isfinite(root[2]).all()


def test_gemm_ex_slots_flags_and_fused_outputs(native_lib):
    """The extras the Newton chain relies on: slot indirection on both operands and on the
    output, the per-matrix skip flag, T = c0 I + c1 D written next to D, and max |D - I|."""
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(8)
    b, n = 3, 200
    Xa = torch.randn(2 * b, n, n, device="cuda", generator=g) / n ** 0.5
    Xb = torch.randn(2 * b, n, n, device="cuda", generator=g) / n ** 0.5
    A, B = _gemm.split3(Xa), _gemm.split3(Xb)
    a_slot = torch.tensor([3, 1, 5], dtype=torch.int32, device="cuda")
    b_slot = torch.tensor([0, 4, 2], dtype=torch.int32, device="cuda")
    d_slot = torch.tensor([2, 0, 1], dtype=torch.int32, device="cuda")
    active = torch.tensor([1, 0, 1], dtype=torch.int32, device="cuda")
    P = _gemm.Planes(b, n, n, "cuda", planes=3)
    T = _gemm.Planes(b, n, n, "cuda", planes=3)
    for X in (P, T):
        for t in (X.hi, X.mid, X.lo):
            t.zero_()
    D = torch.full((b, n, n), 7.0, device="cuda")
    dev = torch.zeros(b, device="cuda")
    _gemm.gemm_ex(A, B, alpha=0.5, D=D, P=P, T=T, t_c0=1.25, t_c1=-0.25, maxdev=dev,
                  a_slot=a_slot, b_slot=b_slot, d_slot=d_slot, active=active, batch=b)
    torch.cuda.synchronize()
    assert native_lib.qt_device_error(1) == 0
    eye = torch.eye(n, device="cuda", dtype=torch.float64)
    for m in range(b):
        want = 0.5 * (Xa[int(a_slot[m])].double() @ Xb[int(b_slot[m])].double())
        out = int(d_slot[m])
        if int(active[m]) == 0:
            assert bool((D[out] == 7.0).all()) and float(P.to_float()[out].abs().max()) == 0.0 and float(dev[m]) == 0.0
            continue
        assert rel(D[out], want) < 1e-5
        assert torch.equal(P.to_float()[out], D[out])                     # three planes carry the fp32 value exactly
        assert rel(T.to_float()[m], 1.25 * eye - 0.25 * want) < 1e-5    # T is stored by matrix number
        assert abs(float(dev[m]) - float((want - eye).abs().max())) < 1e-5


@pytest.mark.parametrize("bn", [128, 256])
def test_both_tile_widths_give_the_same_product(native_lib, bn):
    from optimizers import _gemm
    g = torch.Generator(device="cuda").manual_seed(9)
    A = torch.randn(40, 300, 200, device="cuda", generator=g)
    B = torch.randn(40, 200, 336, device="cuda", generator=g)
    native_lib.qt_gemm_force_tile(bn)
    try:
        D, P = _gemm.matmul(_gemm.split(A), _gemm.split(B), want_planes=True)
        torch.cuda.synchronize()
    finally:
        native_lib.qt_gemm_force_tile(-1)
    assert native_lib.qt_device_error(1) == 0
    ref = A.double() @ B.double()
    assert rel(D, ref) < 1e-5 and rel(P.to_float(), ref) < 2e-5
