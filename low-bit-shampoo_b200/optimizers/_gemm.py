"""Host wrappers of the tcgen05 matrix-product kernels (qt_split_bf16, qt_gemm_bf16x3).

A `Planes` object is an fp32 matrix batch carried as two bf16 planes (hi, lo) with a row
pitch that is a multiple of 16 elements, the operand format of the kernel.  `matmul`
multiplies two such batches with any combination of transposes without moving data: a
transposed operand is presented to the kernel as an MN-major tile.
"""
import ctypes as ct

import torch

import qtensor.functional as F


def _ptr(t):
    return None if t is None else ct.c_void_p(t.data_ptr())


def _pitch(cols):
    return (cols + 15) // 16 * 16       # 32-byte rows: TMA needs 16, the 256-bit epilogue stores 32


class Planes:
    """(batch, rows, cols) fp32 values as bf16 hi/lo planes of pitch `ld`.

    `offset` (elements) selects a sub-matrix of a parent's storage: window() shares memory."""

    def __init__(self, batch, rows, cols, device, _share=None, planes=2):
        self.batch, self.rows, self.cols = batch, rows, cols
        self.mid = None
        if _share is not None:
            self.hi, self.lo, self.ld, self.stride, self.offset = _share[:5]
            self.mid = _share[5] if len(_share) > 5 else None
            return
        self.ld = _pitch(cols)
        self.stride = rows * self.ld
        self.offset = 0
        buf = torch.empty(planes, batch, self.stride, dtype=torch.bfloat16, device=device)
        self.hi, self.lo = buf[0], buf[planes - 1]
        if planes == 3:
            self.mid = buf[1]

    def window(self, row0, col0, rows, cols):
        """Planes of the sub-matrix [row0:row0+rows, col0:col0+cols]; col0 must be a multiple of 8."""
        assert col0 % 8 == 0 and row0 + rows <= self.rows and col0 + cols <= self.cols
        return Planes(self.batch, rows, cols, self.hi.device,
                      _share=(self.hi, self.lo, self.ld, self.stride, self.offset + row0 * self.ld + col0, self.mid))

    def ptr_hi(self):
        return ct.c_void_p(self.hi.data_ptr() + 2 * self.offset)

    def ptr_lo(self):
        return ct.c_void_p(self.lo.data_ptr() + 2 * self.offset)

    def ptr_mid(self):
        return None if self.mid is None else ct.c_void_p(self.mid.data_ptr() + 2 * self.offset)

    def to_float(self):
        n = (self.rows - 1) * self.ld + self.cols
        idx = self.hi[:, self.offset: self.offset + n].float() + self.lo[:, self.offset: self.offset + n].float()
        if self.mid is not None:
            idx = (self.hi[:, self.offset: self.offset + n].float() + self.mid[:, self.offset: self.offset + n].float()) + \
                self.lo[:, self.offset: self.offset + n].float()
        full = torch.zeros(self.batch, self.rows * self.ld, device=idx.device)
        full[:, :n] = idx
        return full.view(self.batch, self.rows, self.ld)[:, :, : self.cols]


def split3(X):
    """fp32 (batch, rows, cols) tensor -> three-plane Planes (hi, mid, lo; 24 significant bits)."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, r, c = X.shape
    P = Planes(b, r, c, X.device, planes=3)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16_3(_ptr(X), X.stride(1), X.stride(0), r, c, b, P.ptr_hi(), _ptr(P.mid), P.ptr_lo(),
                                   P.ld, P.stride, F._stream(X))
    F._check(rc, "split_bf16_3")
    return P


def split(X):
    """fp32 (batch, rows, cols) tensor (last dim contiguous) -> Planes."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, r, c = X.shape
    P = Planes(b, r, c, X.device)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16(_ptr(X), X.stride(1), X.stride(0), r, c, b, P.ptr_hi(), P.ptr_lo(), P.ld, P.stride,
                                 F._stream(X))
    F._check(rc, "split_bf16")
    return P


def split_rows(X, index=None, scale=None):
    """Planes of the matrices whose row i is scale[b, i] * X[b, index[b, i], :] (qt_split_bf16_rows).
    X: fp32 (batch, R, cols); index: int64 (batch, rows) or None; scale: fp32 (batch, rows) or None."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, R, c = X.shape
    rows = index.shape[1] if index is not None else R
    if index is not None:
        assert index.dtype == torch.int64 and index.shape[0] == b and index.stride(1) == 1
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.shape == (b, rows) and scale.stride(1) == 1
    P = Planes(b, rows, c, X.device)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16_rows(_ptr(X), X.stride(1), X.stride(0), rows, c, b,
                                      _ptr(index), index.stride(0) if index is not None else 0,
                                      _ptr(scale), scale.stride(0) if scale is not None else 0,
                                      P.ptr_hi(), P.ptr_lo(), P.ld, P.stride, F._stream(X))
    F._check(rc, "split_bf16_rows")
    return P


def matmul(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, out=None, want_planes=False,
           want_float=True, out_planes=None):
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
    P = out_planes if out_planes is not None else (Planes(b, M, N, dev) if want_planes else None)
    if P is not None:
        assert P.rows == M and P.cols == N and P.batch == b
    if C is not None:
        assert C.stride(2) == 1
    # kernel view: A logically M x K (a_mn: stored [K][M]); B logically N x K (b_mn: stored [K][N])
    a_mn = 1 if trans_a else 0
    b_mn = 0 if trans_b else 1
    if A.mid is not None or B.mid is not None:
        assert A.mid is not None and B.mid is not None
        if P is not None:
            # fp32-level product whose result is also handed on as three planes
            if out_planes is None:
                P = Planes(b, M, N, dev, planes=3)
            assert P.mid is not None
            gemm_ex(A, B, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta, C=C, D=D, P=P)
            return D, P
        assert D is not None
        with torch.cuda.device(dev):
            rc = F.lib.qt_gemm_bf16x6(
                A.ptr_hi(), A.ptr_mid(), A.ptr_lo(), A.ld, A.stride, a_mn,
                B.ptr_hi(), B.ptr_mid(), B.ptr_lo(), B.ld, B.stride, b_mn,
                M, N, K, b, float(alpha), float(beta),
                _ptr(C), C.stride(1) if C is not None else 0, C.stride(0) if C is not None else 0,
                _ptr(D), D.stride(1), D.stride(0), F._stream(A.hi))
        F._check(rc, "gemm_bf16x6")
        return D, None
    with torch.cuda.device(dev):
        rc = F.lib.qt_gemm_bf16x3(
            A.ptr_hi(), A.ptr_lo(), A.ld, A.stride, a_mn,
            B.ptr_hi(), B.ptr_lo(), B.ld, B.stride, b_mn,
            M, N, K, b, float(alpha), float(beta),
            _ptr(C), C.stride(1) if C is not None else 0, C.stride(0) if C is not None else 0,
            _ptr(D), D.stride(1) if D is not None else 0, D.stride(0) if D is not None else 0,
            P.ptr_hi() if P else None, P.ptr_lo() if P else None, P.ld if P else 0, P.stride if P else 0,
            F._stream(A.hi))
    F._check(rc, "gemm_bf16x3")
    return D, P


def matmul_q4(A, B, code, out, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, old=None):
    """out <- quantize(alpha * op(A) @ op(B) + beta * dequantize(old)) on 4-bit block-64 state.

    A, B: Planes (both two-plane or both three-plane) of a square product (b, n, n), n a multiple of 16.  `out` and
    `old` are (codes uint8 (b, row_bytes), absmax fp32 (b, n*nb), diag fp32 (b, n) or None);
    `old=None` drops the C operand, `old is out` updates in place.  Same bytes as
    dequantize -> six-product GEMM -> quantize, without an fp32 copy of the state in HBM
    (qt_gemm_bf16x6_q4).
    """
    M = A.cols if trans_a else A.rows
    K = A.rows if trans_a else A.cols
    Kb = B.cols if trans_b else B.rows
    N = B.rows if trans_b else B.cols
    assert K == Kb and A.batch == B.batch and M == N and (A.mid is None) == (B.mid is None)
    b = A.batch
    var, absmax, diag = out
    assert var.dtype == torch.uint8 and var.dim() == 2 and var.shape[0] == b and var.stride(1) == 1
    assert absmax.dim() == 2 and absmax.stride(1) == 1 and (diag is None or diag.stride(1) == 1)
    ovar = oabs = odiag = None
    if old is not None:
        ovar, oabs, odiag = old
        assert ovar.stride(0) == var.stride(0) and oabs.stride(0) == absmax.stride(0)
        assert odiag is None or diag is None or odiag.stride(0) == diag.stride(0)
    tail = (N, K, b, float(alpha), float(beta), _ptr(code),
            _ptr(ovar), _ptr(oabs), _ptr(odiag), _ptr(var), _ptr(absmax), _ptr(diag),
            var.stride(0), absmax.stride(0),
            (diag if diag is not None else odiag).stride(0) if (diag is not None or odiag is not None) else 0,
            F._stream(var))
    with torch.cuda.device(var.device):
        if A.mid is not None:
            rc = F.lib.qt_gemm_bf16x6_q4(
                A.ptr_hi(), _ptr(A.mid), A.ptr_lo(), A.ld, A.stride, 1 if trans_a else 0,
                B.ptr_hi(), _ptr(B.mid), B.ptr_lo(), B.ld, B.stride, 0 if trans_b else 1, *tail)
        else:
            rc = F.lib.qt_gemm_bf16x3_q4(
                A.ptr_hi(), A.ptr_lo(), A.ld, A.stride, 1 if trans_a else 0,
                B.ptr_hi(), B.ptr_lo(), B.ld, B.stride, 0 if trans_b else 1, *tail)
    F._check(rc, "gemm_q4")


def gemm_ex(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, D=None, P=None, T=None, t_c0=0.0, t_c1=0.0,
            maxdev=None, a_slot=None, b_slot=None, d_slot=None, active=None, batch=None):
    """General product (qt_gemm_ex): A, B are Planes (two- or three-plane, possibly holding more
    entries than `batch` when slot arrays select among them); results go to the fp32 tensor D and / or
    the Planes P, and optionally T = t_c0 * I + t_c1 * result (three planes, indexed by matrix number).
    maxdev: fp32 (batch,) combined with max |result - I|; *_slot, active: int32 (batch,) device tensors."""
    from qtensor.cextension import GemmDesc
    M = A.cols if trans_a else A.rows
    K = A.rows if trans_a else A.cols
    N = B.rows if trans_b else B.cols
    b = batch if batch is not None else A.batch
    d = GemmDesc()
    ip = lambda t: None if t is None else t.data_ptr()
    po = lambda X, t: None if t is None else t.data_ptr() + 2 * X.offset
    d.A[0], d.A[1], d.A[2] = po(A, A.hi), po(A, A.mid), po(A, A.lo)
    d.B[0], d.B[1], d.B[2] = po(B, B.hi), po(B, B.mid), po(B, B.lo)
    d.lda, d.strideA, d.a_mn, d.a_entries = A.ld, A.stride, 1 if trans_a else 0, A.batch
    d.ldb, d.strideB, d.b_mn, d.b_entries = B.ld, B.stride, 0 if trans_b else 1, B.batch
    d.M, d.N, d.K, d.batch, d.alpha, d.beta = M, N, K, b, float(alpha), float(beta)
    if C is not None:
        d.C, d.ldc, d.strideC = C.data_ptr(), C.stride(1), C.stride(0)
    if D is not None:
        d.D, d.ldd, d.strideD = D.data_ptr(), D.stride(1), D.stride(0)
    for X, field in ((P, d.P), (T, d.T)):
        if X is not None:
            field[0], field[1], field[2] = po(X, X.hi), po(X, X.mid), po(X, X.lo)
            d.ldp, d.strideP = X.ld, X.stride
    d.t_c0, d.t_c1 = float(t_c0), float(t_c1)
    d.maxdev, d.a_slot, d.b_slot, d.d_slot, d.active = ip(maxdev), ip(a_slot), ip(b_slot), ip(d_slot), ip(active)
    with torch.cuda.device(A.hi.device):
        rc = F.lib.qt_gemm_ex(ct.byref(d), F._stream(A.hi))
    F._check(rc, "gemm_ex")
