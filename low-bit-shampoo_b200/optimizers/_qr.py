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


USE_TENSOR_CORES = False     # trailing updates: rank-32 products are memory-bound; fp32 library products are faster here


def _reflect(lib, stream, Vk, Tk, target, target_planes, transpose_t):
    """target <- (I - Vk T Vk^T) target (or with T^T), fp32 in place, planes kept in step."""
    from optimizers import _gemm
    if target_planes is None:
        W = torch.bmm(Vk.transpose(1, 2), target)
        W = torch.bmm(Tk.transpose(1, 2) if transpose_t else Tk, W)
        target.baddbmm_(Vk, W, alpha=-1.0)
        return
    Pv = _gemm.split(Vk)
    W, _ = _gemm.matmul(Pv, target_planes, trans_a=True)                   # Vk^T target, (w x t)
    W = torch.bmm(Tk.transpose(1, 2) if transpose_t else Tk, W)
    _gemm.matmul(Pv, _gemm.split(W), alpha=-1.0, beta=1.0, C=target, out=target, out_planes=target_planes)


def householder_q(X):
    """Q of the QR factorisation of each X[b] (X: (B, n, n) fp32 CUDA, overwritten)."""
    B, n, _ = X.shape
    if (not X.is_cuda) or n > MAX_ORDER or n < 2 * PANEL:
        return torch.linalg.qr(X).Q
    F._require_lib(X)
    X = X.contiguous()
    lib = F.lib
    from optimizers import _gemm
    tc = USE_TENSOR_CORES
    panels = list(range(0, n, PANEL))
    V = torch.zeros(B, n, n, dtype=torch.float32, device=X.device)
    T = torch.empty(B, len(panels), PANEL, PANEL, dtype=torch.float32, device=X.device)
    stream = F._stream(X)
    with torch.cuda.device(X.device):
        Xp = _gemm.split(X) if tc else None
        for k, j0 in enumerate(panels):
            w = min(PANEL, n - j0)
            rc = lib.qt_householder_panel(_ptr(X), n * n, n, B, j0, w, _ptr(V), n * n,
                                          _ptr(T[:, k]), len(panels) * PANEL * PANEL, stream)
            F._check(rc, "householder panel")
            if j0 + w < n:
                m, t = n - j0, n - j0 - w
                _reflect(lib, stream, V[:, j0:, j0:j0 + w], T[:, k, :w, :w], X[:, j0:, j0 + w:],
                         Xp.window(j0, j0 + w, m, t) if tc else None, transpose_t=True)
        Q = torch.eye(n, dtype=torch.float32, device=X.device).expand(B, n, n).contiguous()
        Qp = _gemm.split(Q) if tc else None
        for k in reversed(range(len(panels))):
            j0 = panels[k]
            w = min(PANEL, n - j0)
            m = n - j0
            _reflect(lib, stream, V[:, j0:, j0:j0 + w], T[:, k, :w, :w], Q[:, j0:, j0:],
                     Qp.window(j0, j0, m, m) if tc else None, transpose_t=False)
    return Q
