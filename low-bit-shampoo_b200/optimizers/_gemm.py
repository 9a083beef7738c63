"""Host wrappers of the tcgen05 matrix-product kernels (qt_split_bf16, qt_gemm_bf16x3).

A `Planes` object is an fp32 matrix batch carried as two bf16 planes (hi, lo) with a row
pitch that is a multiple of 8 elements, the operand format of the kernel.  `matmul`
multiplies two such batches with any combination of transposes without moving data: a
transposed operand is presented to the kernel as an MN-major tile.
"""
import ctypes as ct

import torch

import qtensor.functional as F


def _ptr(t):
    return None if t is None else ct.c_void_p(t.data_ptr())


def _pitch(cols):
    return (cols + 7) // 8 * 8


class Planes:
    """(batch, rows, cols) fp32 values as bf16 hi/lo planes of pitch `ld`."""

    def __init__(self, batch, rows, cols, device):
        self.batch, self.rows, self.cols = batch, rows, cols
        self.ld = _pitch(cols)
        self.rows_alloc = rows
        self.stride = self.rows_alloc * self.ld
        buf = torch.empty(2, batch, self.stride, dtype=torch.bfloat16, device=device)
        self.hi, self.lo = buf[0], buf[1]

    def to_float(self):
        v = (self.hi.float() + self.lo.float()).view(self.batch, self.rows_alloc, self.ld)
        return v[:, : self.rows, : self.cols]


def split(X):
    """fp32 (batch, rows, cols) tensor (last dim contiguous) -> Planes."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, r, c = X.shape
    P = Planes(b, r, c, X.device)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16(_ptr(X), X.stride(1), X.stride(0), r, c, b, _ptr(P.hi), _ptr(P.lo), P.ld, P.stride,
                                 F._stream(X))
    F._check(rc, "split_bf16")
    return P


def matmul(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, out=None, want_planes=False,
           want_float=True):
    """alpha * op(A) @ op(B) + beta * C for batches held as Planes.

    A holds (b, M, K) (or (b, K, M) with trans_a); B holds (b, K, N) (or (b, N, K) with
    trans_b).  Returns (fp32 tensor or None, Planes or None).
    """
    M = A.cols if trans_a else A.rows
    K = A.rows if trans_a else A.cols
    Kb = B.cols if trans_b else B.rows
    N = B.rows if trans_b else B.cols
    assert K == Kb and A.batch == B.batch
    b = A.batch
    dev = A.hi.device
    D = None
    if want_float:
        D = out if out is not None else torch.empty(b, M, N, dtype=torch.float32, device=dev)
        assert D.stride(2) == 1
    P = Planes(b, M, N, dev) if want_planes else None
    if C is not None:
        assert C.stride(2) == 1
    # kernel view: A logically M x K (a_mn: stored [K][M]); B logically N x K (b_mn: stored [K][N])
    a_mn = 1 if trans_a else 0
    b_mn = 0 if trans_b else 1
    with torch.cuda.device(dev):
        rc = F.lib.qt_gemm_bf16x3(
            _ptr(A.hi), _ptr(A.lo), A.ld, A.stride, a_mn,
            _ptr(B.hi), _ptr(B.lo), B.ld, B.stride, b_mn,
            M, N, K, b, float(alpha), float(beta),
            _ptr(C), C.stride(1) if C is not None else 0, C.stride(0) if C is not None else 0,
            _ptr(D), D.stride(1) if D is not None else 0, D.stride(0) if D is not None else 0,
            _ptr(P.hi) if P else None, _ptr(P.lo) if P else None, P.ld if P else 0, P.stride if P else 0,
            F._stream(A.hi))
    F._check(rc, "gemm_bf16x3")
    return D, P
