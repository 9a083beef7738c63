"""Batched Householder QR (panel kernel through the C ABI + batched updates) against
torch.linalg.qr on the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4


def check(X):
    from optimizers._qr import householder_q
    Q = householder_q(X.clone())
    Qt = torch.linalg.qr(X).Q
    n = X.shape[-1]
    eye = torch.eye(n, device=X.device)
    orth = float(((Q.transpose(1, 2) @ Q - eye).flatten(1).norm(dim=1)).max())
    assert orth < 5e-5 * n ** 0.5, orth
    # Q^T X must be upper triangular (same column space, nested)
    R = Q.transpose(1, 2) @ X
    low = float((torch.tril(R, -1).flatten(1).norm(dim=1) / X.flatten(1).norm(dim=1)).max())
    assert low < 1e-5, low
    return Q, Qt


@pytest.mark.parametrize("n", [64, 96, 100, 672, 768, 1000, 1104, 1200])
def test_full_rank_matches_lapack_convention(native_lib, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    X = torch.randn(3, n, n, device="cuda", generator=g)
    Q, Qt = check(X)
    rel = float(((Q - Qt).flatten(1).norm(dim=1) / Qt.flatten(1).norm(dim=1)).max())
    assert rel < TOL, rel


def test_statistic_like_input(native_lib):
    """X = L V^T with L symmetric PSD of wide spectrum, as in the eigenbasis refresh."""
    n = 768
    g = torch.Generator(device="cuda").manual_seed(1)
    U = torch.linalg.qr(torch.randn(n, n, device="cuda", generator=g, dtype=torch.float64)).Q
    lam = torch.logspace(-4, 0, n, device="cuda", dtype=torch.float64)
    L = ((U * lam) @ U.T).float()
    X = torch.stack([L, L @ L, L + 0.1 * torch.eye(n, device="cuda")])
    check(X)


def test_rank_deficient_input_stays_orthonormal(native_lib):
    n = 256
    g = torch.Generator(device="cuda").manual_seed(2)
    G = torch.randn(2, n, 40, device="cuda", generator=g)
    X = G @ G.transpose(1, 2)                      # rank 40
    X[:, :, 5] = 0.0                               # an exactly zero column
    check(X)


@pytest.mark.parametrize("n,batch", [(768, 3), (1200, 2), (400, 5)])
def test_lookahead_orchestration_gives_the_same_q(native_lib, n, batch):
    """The optional orchestration (far update split into the next block's columns and a remainder on
    a side stream, Q accumulated forwards on a second one, side products on a capped grid) computes
    the same factorisation in another order of operations: Q agrees to rounding, stays orthonormal,
    and the device status stays clean."""
    from optimizers import _qr
    g = torch.Generator(device="cuda").manual_seed(n)
    X = torch.randn(batch, n, n, device="cuda", generator=g)
    base = _qr.householder_q(X.clone())
    old = (_qr.LOOKAHEAD, _qr.FORWARD_Q)
    try:
        for forward in (False, True):
            _qr.LOOKAHEAD, _qr.FORWARD_Q = True, forward
            Q = _qr.householder_q(X.clone())
            torch.cuda.synchronize()
            assert native_lib.qt_device_error(1) == 0
            assert float((Q - base).norm() / base.norm()) < 1e-5
            eye = torch.eye(n, device="cuda")
            assert float((Q.transpose(1, 2) @ Q - eye).abs().max()) < 1e-4
    finally:
        _qr.LOOKAHEAD, _qr.FORWARD_Q = old


@pytest.mark.parametrize("n", [768, 1200])
def test_both_tall_panel_kernels_agree(native_lib, n):
    """Panels of more than 640 rows are factored with two columns per warp by default and with one
    column per warp on request: same conventions, Q equal to rounding."""
    from optimizers import _qr
    g = torch.Generator(device="cuda").manual_seed(3 * n)
    X = torch.randn(2, n, n, device="cuda", generator=g)
    Q0 = _qr.householder_q(X.clone())
    try:
        native_lib.qt_panel_force_form(1)
        Q1 = _qr.householder_q(X.clone())
    finally:
        native_lib.qt_panel_force_form(0)
    torch.cuda.synchronize()
    assert native_lib.qt_device_error(1) == 0
    assert float((Q0 - Q1).norm() / Q1.norm()) < 1e-5
    check(X)


def test_orders_beyond_the_panel_kernel_fall_back_with_a_warning(native_lib):
    """A panel of more than 1216 rows does not fit one SM's shared memory: such orders go to
    torch.linalg.qr, and say so once."""
    from optimizers import _qr
    _qr._WARNED_LARGE = False
    X = torch.randn(1, _qr.MAX_ORDER + 16, _qr.MAX_ORDER + 16, device="cuda")
    with pytest.warns(UserWarning, match="torch.linalg.qr"):
        Q = _qr.householder_q(X.clone())
    assert float((Q - torch.linalg.qr(X).Q).abs().max()) == 0.0
