"""Batched Householder QR (Q factor only) for a stack of square matrices.

Replaces the per-matrix torch.linalg.qr of the reference's eigenbasis refresh
(qtensor/utils.py:157).  Blocked compact-WY algorithm with 32-column panels: the panel
factorisation of every matrix of the batch is one launch of the library's
qt_householder_panel kernel; the trailing update  A <- (I - V T^T V^T) A  and the backward
accumulation  Q <- (I - V T V^T) Q  are batched products.  Sign conventions are LAPACK's,
so Q agrees with torch.linalg.qr's up to rounding on full-rank input.
"""
import ctypes as ct

import torch

import qtensor.functional as F

PANEL = 32
MAX_ORDER = 1700            # the panel kernel keeps a (rows x 32) panel in shared memory


def _ptr(t):
    return ct.c_void_p(t.data_ptr())


def householder_q(X):
    """Q of the QR factorisation of each X[b] (X: (B, n, n) fp32 CUDA, overwritten)."""
    B, n, _ = X.shape
    if (not X.is_cuda) or n > MAX_ORDER or n < 2 * PANEL:
        return torch.linalg.qr(X).Q
    F._require_lib(X)
    X = X.contiguous()
    lib = F.lib
    panels = list(range(0, n, PANEL))
    V = torch.zeros(B, n, n, dtype=torch.float32, device=X.device)
    T = torch.empty(B, len(panels), PANEL, PANEL, dtype=torch.float32, device=X.device)
    stream = F._stream(X)
    with torch.cuda.device(X.device):
        for k, j0 in enumerate(panels):
            w = min(PANEL, n - j0)
            rc = lib.qt_householder_panel(_ptr(X), n * n, n, B, j0, w, _ptr(V), n * n,
                                          _ptr(T[:, k]), len(panels) * PANEL * PANEL, stream)
            F._check(rc, "householder panel")
            if j0 + w < n:
                Vk = V[:, j0:, j0:j0 + w]
                trail = X[:, j0:, j0 + w:]
                W = torch.bmm(Vk.transpose(1, 2), trail)
                W = torch.bmm(T[:, k, :w, :w].transpose(1, 2), W)
                trail.baddbmm_(Vk, W, alpha=-1.0)
        Q = torch.eye(n, dtype=torch.float32, device=X.device).expand(B, n, n).contiguous()
        for k in reversed(range(len(panels))):
            j0 = panels[k]
            w = min(PANEL, n - j0)
            Vk = V[:, j0:, j0:j0 + w]
            sub = Q[:, j0:, j0:]
            W = torch.bmm(Vk.transpose(1, 2), sub)
            W = torch.bmm(T[:, k, :w, :w], W)
            sub.baddbmm_(Vk, W, alpha=-1.0)
    return Q
