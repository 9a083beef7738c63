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
