"""Host wrappers of the tcgen05 matrix-product kernels.

A `Planes` object is a batch of fp32 matrices in the operand format of the product kernel:
row pitch a multiple of 16 elements, one of three encodings

  * scaled fp16, two planes (the default of split()): entry = x * 2^(exp[b] + exp0) as
    hi = fp16(.), lo = fp16(. - hi) - 22 significant bits; the per-matrix exponent exp[b] is
    chosen from the matrix's largest magnitude so that scaled entries stay below 2^tmax.
    Three MMAs per k-slice (hi*hi + hi*lo + lo*hi) on fp16 operands, partial sums of 128 k
    promoted to fp32 registers: products agree with an fp32 library product to ~1e-6;
  * bf16, two planes (split_bf16()): 16 significant bits, no scaling - the format of the
    plain C entry points qt_split_bf16 / qt_gemm_bf16x3;
  * bf16, three planes (split3()): 24 significant bits, six MMAs per k-slice - used by the
    Schur-Newton chain, whose iterates have no usable a-priori bound.

`matmul` multiplies two such batches with any combination of transposes without moving
data: a transposed operand is presented to the kernel as an MN-major tile.
"""
import ctypes as ct
import math

import torch

import qtensor.functional as F

FP16_PLANES = True          # split() produces scaled fp16 planes (False: bf16 planes, 16 significant bits)
SPLIT_TARGET = 9            # scaled entries of a freshly split matrix stay below 2^9 (headroom for in-place updates)
CHAIN_K = 2                 # k-blocks (of 64) per accumulation chain of fp16-plane products
F16_MAX_EXP = 15            # fp16 holds magnitudes below 2^16; plane outputs are placed below 2^15


def _ptr(t):
    return None if t is None else ct.c_void_p(t.data_ptr())


def _ceil_log2(x):
    return int(math.ceil(math.log2(max(float(x), 1e-30))))


def _pitch(cols):
    return (cols + 15) // 16 * 16       # 32-byte rows: TMA needs 16, the 256-bit epilogue stores 32


class Planes:
    """(batch, rows, cols) fp32 values as 16-bit planes of pitch `ld` (see the module docstring).

    `offset` (elements) selects a sub-matrix of a parent's storage: window() shares memory,
    exponents included."""

    def __init__(self, batch, rows, cols, device, _share=None, planes=2, f16=False, exp=None, exp0=0, tmax=None):
        self.batch, self.rows, self.cols = batch, rows, cols
        self.mid = None
        self.f16, self.exp, self.exp0, self.tmax = f16, exp, exp0, tmax
        if _share is not None:
            self.hi, self.lo, self.ld, self.stride, self.offset = _share[:5]
            self.mid = _share[5] if len(_share) > 5 else None
            return
        assert not (f16 and planes == 3)
        self.ld = _pitch(cols)
        self.stride = rows * self.ld
        self.offset = 0
        buf = torch.empty(planes, batch, self.stride, dtype=torch.float16 if f16 else torch.bfloat16, device=device)
        self.hi, self.lo = buf[0], buf[planes - 1]
        if planes == 3:
            self.mid = buf[1]

    def window(self, row0, col0, rows, cols):
        """Planes of the sub-matrix [row0:row0+rows, col0:col0+cols]; col0 must be a multiple of 8."""
        assert col0 % 8 == 0 and row0 + rows <= self.rows and col0 + cols <= self.cols
        return Planes(self.batch, rows, cols, self.hi.device,
                      _share=(self.hi, self.lo, self.ld, self.stride, self.offset + row0 * self.ld + col0, self.mid),
                      f16=self.f16, exp=self.exp, exp0=self.exp0, tmax=self.tmax)

    def ptr_hi(self):
        return ct.c_void_p(self.hi.data_ptr() + 2 * self.offset)

    def ptr_lo(self):
        return ct.c_void_p(self.lo.data_ptr() + 2 * self.offset)

    def ptr_mid(self):
        return None if self.mid is None else ct.c_void_p(self.mid.data_ptr() + 2 * self.offset)

    def to_float(self):
        n = (self.rows - 1) * self.ld + self.cols
        sl = slice(self.offset, self.offset + n)
        val = self.hi[:, sl].float() + self.lo[:, sl].float()
        if self.mid is not None:
            val = (self.hi[:, sl].float() + self.mid[:, sl].float()) + self.lo[:, sl].float()
        if self.f16:
            e = torch.full((self.batch,), float(self.exp0), device=val.device)
            if self.exp is not None:
                e = e + self.exp.float()
            val = val * torch.exp2(-e).unsqueeze(1)
        full = torch.zeros(self.batch, self.rows * self.ld, device=val.device)
        full[:, :n] = val
        return full.view(self.batch, self.rows, self.ld)[:, :, : self.cols]


class StateOperand:
    """A product operand that stays 4-bit state: `batch` square matrices of order n, matrix m being
    slot slots[m] of an arena (codes uint8 (count, row_bytes), absmax fp32 (count, n*nb), diag fp32
    (count, n) or None).  The product kernel's converter warps dequantize it tile by tile in
    shared memory (qt_gemm_ex, aq_* / bq_*); only the per-matrix plane exponents are computed
    beforehand, from the block scales and the diagonal (qt_state_exponents)."""

    f16, mid, exp0, offset = True, None, 0, 0

    def __init__(self, var, absmax, diag, code, n, slots, target=None):
        self.var, self.absmax, self.diag, self.code, self.slots = var, absmax, diag, code, slots
        self.rows = self.cols = n
        self.batch = slots.numel()
        self.tmax = SPLIT_TARGET if target is None else target
        self.hi = var                                       # device / stream anchor
        self.exp = torch.empty(self.batch, dtype=torch.int32, device=var.device)
        with torch.cuda.device(var.device):
            rc = F.lib.qt_state_exponents(_ptr(absmax), absmax.stride(0), absmax.shape[1],
                                          _ptr(diag), diag.stride(0) if diag is not None else 0, n,
                                          _ptr(slots), self.batch, self.tmax, _ptr(self.exp), F._stream(var))
        F._check(rc, "state exponents")


def split3(X):
    """fp32 (batch, rows, cols) tensor -> three-plane bf16 Planes (hi, mid, lo; 24 significant bits)."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, r, c = X.shape
    P = Planes(b, r, c, X.device, planes=3)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16_3(_ptr(X), X.stride(1), X.stride(0), r, c, b, P.ptr_hi(), _ptr(P.mid), P.ptr_lo(),
                                   P.ld, P.stride, F._stream(X))
    F._check(rc, "split_bf16_3")
    return P


def split_bf16(X):
    """fp32 (batch, rows, cols) tensor (last dim contiguous) -> two-plane bf16 Planes."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, r, c = X.shape
    P = Planes(b, r, c, X.device)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16(_ptr(X), X.stride(1), X.stride(0), r, c, b, P.ptr_hi(), P.ptr_lo(), P.ld, P.stride,
                                 F._stream(X))
    F._check(rc, "split_bf16")
    return P


def _split_f16(X, index, scale, target, bound):
    """`bound`: None - each matrix's largest magnitude is measured (one extra pass over X);
    a float - an a-priori bound on every entry (one exponent for the whole batch, no pass);
    an fp32 tensor (batch,) - per-matrix bounds known on the device (no pass)."""
    b, R, c = X.shape
    rows = index.shape[1] if index is not None else R
    amax = exp = None
    compute, exp0 = 0, target
    if bound is None:
        scratch = torch.empty(2, b, dtype=torch.int32, device=X.device)  # [0]: amax (as float bits), [1]: exponents
        amax, exp, compute = scratch[0], scratch[1], 1
    elif torch.is_tensor(bound):
        assert bound.dtype == torch.float32 and bound.shape == (b,) and bound.is_contiguous()
        amax, exp = bound, torch.empty(b, dtype=torch.int32, device=X.device)
    else:
        exp0 = target - _ceil_log2(bound)
    P = Planes(b, rows, c, X.device, f16=True, exp=exp, exp0=0 if exp is not None else exp0, tmax=target)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_f16(_ptr(X), X.stride(1), X.stride(0), rows, c, b,
                                _ptr(index), index.stride(0) if index is not None else 0,
                                _ptr(scale), scale.stride(0) if scale is not None else 0,
                                _ptr(amax), compute, None, exp0, _ptr(exp),
                                P.ptr_hi(), P.ptr_lo(), P.ld, P.stride, F._stream(X))
    F._check(rc, f"split_f16 ({b} x {rows}x{c})")
    return P


def split(X, target=None, bound=None):
    """fp32 (batch, rows, cols) tensor (last dim contiguous) -> Planes (scaled fp16 unless FP16_PLANES is off).
    `bound`: see _split_f16."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    if not FP16_PLANES:
        return split_bf16(X)
    return _split_f16(X, None, None, SPLIT_TARGET if target is None else target, bound)


def split_rows(X, index=None, scale=None, target=None, bound=None):
    """Planes of the matrices whose row i is scale[b, i] * X[b, index[b, i], :].
    X: fp32 (batch, R, cols); index: int64 (batch, rows) or None; scale: fp32 (batch, rows) or None;
    `bound` on the SCALED rows: see _split_f16."""
    assert X.dim() == 3 and X.dtype == torch.float32 and X.stride(2) == 1
    b, R, c = X.shape
    rows = index.shape[1] if index is not None else R
    if index is not None:
        assert index.dtype == torch.int64 and index.shape[0] == b and index.stride(1) == 1
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.shape == (b, rows) and scale.stride(1) == 1
    if FP16_PLANES:
        return _split_f16(X, index, scale, SPLIT_TARGET if target is None else target, bound)
    P = Planes(b, rows, c, X.device)
    with torch.cuda.device(X.device):
        rc = F.lib.qt_split_bf16_rows(_ptr(X), X.stride(1), X.stride(0), rows, c, b,
                                      _ptr(index), index.stride(0) if index is not None else 0,
                                      _ptr(scale), scale.stride(0) if scale is not None else 0,
                                      P.ptr_hi(), P.ptr_lo(), P.ld, P.stride, F._stream(X))
    F._check(rc, "split_bf16_rows")
    return P


def matmul(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, out=None, want_planes=False,
           want_float=True, out_planes=None, out_bound=None, max_ctas=0):
    """alpha * op(A) @ op(B) + beta * C for batches held as Planes.

    A holds (b, M, K) (or (b, K, M) with trans_a); B holds (b, K, N) (or (b, N, K) with
    trans_b).  Returns (fp32 tensor or None, Planes or None).  Plane output of an fp16-plane
    product: into `out_planes` (its exponents are kept - the caller vouches that the result fits),
    or freshly allocated with exponent such that |result| <= out_bound fits if `out_bound` is
    given, else with the worst-case exponent K * max|A| * max|B| * |alpha| (beta must be 0 then).
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
    if C is not None:
        assert C.stride(2) == 1
    if isinstance(A, StateOperand) or isinstance(B, StateOperand):
        assert not trans_a and not trans_b, "an operand from 4-bit state is used as stored (row-major)"
    three = A.mid is not None or B.mid is not None
    f16 = A.f16 or B.f16
    if three:
        assert A.mid is not None and B.mid is not None and not f16
    else:
        assert A.f16 == B.f16, "both operands must use the same plane encoding"
    P = out_planes
    if P is None and want_planes:
        P = Planes(b, M, N, dev, planes=3 if three else 2, f16=f16)
    if P is not None:
        assert P.rows == M and P.cols == N and P.batch == b and P.f16 == f16 and (P.mid is not None) == three
    if not three and not f16 and not (P is None and D is None):
        # plain bf16 two-plane product: the fixed-signature entry point
        a_mn, b_mn = (1 if trans_a else 0), (0 if trans_b else 1)
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
    kw = {}
    if f16 and P is not None:
        if out_planes is not None:
            kw = dict(out_exp=P.exp, out_exp0=P.exp0)
        elif out_bound is not None:
            P.exp, P.exp0, P.tmax = None, F16_MAX_EXP - _ceil_log2(out_bound), F16_MAX_EXP
            kw = dict(out_exp0=P.exp0)
        else:
            assert beta == 0.0 or C is None, "worst-case plane exponents cannot account for a C operand"
            rel = F16_MAX_EXP - _ceil_log2(K) - A.tmax - B.tmax - _ceil_log2(abs(alpha))
            P.exp = torch.empty(b, dtype=torch.int32, device=dev)
            P.exp0, P.tmax = 0, F16_MAX_EXP
            kw = dict(out_rel=1, out_exp0=rel, out_exp_w=P.exp)
    gemm_ex(A, B, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta, C=C, D=D, P=P, max_ctas=max_ctas, **kw)
    return D, P


def matmul_q4(A, B, code, out, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, old=None):
    """out <- quantize(alpha * op(A) @ op(B) + beta * dequantize(old)) on 4-bit block-64 state.

    A, B: Planes of one encoding, of a square product (b, n, n), n a multiple of 16.  `out` and
    `old` are (codes uint8 (b, row_bytes), absmax fp32 (b, n*nb), diag fp32 (b, n) or None);
    `old=None` drops the C operand, `old is out` updates in place.  Same bytes as
    dequantize -> product -> quantize, without an fp32 copy of the state in HBM.
    """
    M = A.cols if trans_a else A.rows
    N = B.rows if trans_b else B.cols
    assert M == N and A.batch == B.batch and (A.mid is None) == (B.mid is None) and A.f16 == B.f16
    b = A.batch
    var, absmax, diag = out
    assert var.dtype == torch.uint8 and var.dim() == 2 and var.shape[0] == b and var.stride(1) == 1
    assert absmax.dim() == 2 and absmax.stride(1) == 1 and (diag is None or diag.stride(1) == 1)
    ovar = oabs = odiag = None
    if old is not None:
        ovar, oabs, odiag = old
        assert ovar.stride(0) == var.stride(0) and oabs.stride(0) == absmax.stride(0)
        assert odiag is None or diag is None or odiag.stride(0) == diag.stride(0)
    sd = (diag if diag is not None else odiag).stride(0) if (diag is not None or odiag is not None) else 0
    gemm_ex(A, B, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta,
            q=dict(code=code, q_in=ovar, absmax_in=oabs, diag_in=odiag, q_out=var, absmax_out=absmax, diag_out=diag,
                   stride_codes=var.stride(0), stride_absmax=absmax.stride(0), stride_diag=sd))


def gemm_ex(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, D=None, P=None, T=None, t_c0=0.0, t_c1=0.0,
            maxdev=None, a_slot=None, b_slot=None, d_slot=None, active=None, batch=None,
            out_exp=None, out_exp0=0, out_rel=0, out_exp_w=None, q=None, max_ctas=0, c_follows_d=False):
    """General product (qt_gemm_ex): A, B are Planes (possibly holding more entries than `batch` when slot
    arrays select among them); results go to the fp32 tensor D and / or the Planes P, optionally
    T = t_c0 * I + t_c1 * result (three bf16 planes, indexed by matrix number), or - with `q` - into
    4-bit state.  maxdev: fp32 (batch,) combined with max |result - I|; *_slot, active: int32 device tensors."""
    from qtensor.cextension import GemmDesc
    M = A.cols if trans_a else A.rows
    K = A.rows if trans_a else A.cols
    N = B.rows if trans_b else B.cols
    b = batch if batch is not None else A.batch
    d = GemmDesc()
    ip = lambda t: None if t is None else t.data_ptr()
    po = lambda X, t: None if t is None else t.data_ptr() + 2 * X.offset
    d.a_mn, d.b_mn = 1 if trans_a else 0, 0 if trans_b else 1
    for X, side in ((A, "a"), (B, "b")):
        if isinstance(X, StateOperand):
            setattr(d, side + "q_codes", ip(X.var)); setattr(d, side + "q_absmax", ip(X.absmax)); setattr(d, side + "q_diag", ip(X.diag))
            setattr(d, side + "q_slots", ip(X.slots)); setattr(d, side + "q_stride_codes", X.var.stride(0))
            setattr(d, side + "q_stride_absmax", X.absmax.stride(0)); setattr(d, side + "q_stride_diag", X.diag.stride(0) if X.diag is not None else 0)
            d.oq_code = ip(X.code)
    if not isinstance(A, StateOperand):
        d.A[0], d.A[1], d.A[2] = po(A, A.hi), po(A, A.mid), po(A, A.lo)
        d.lda, d.strideA, d.a_entries = A.ld, A.stride, A.batch
    if not isinstance(B, StateOperand):
        d.B[0], d.B[1], d.B[2] = po(B, B.hi), po(B, B.mid), po(B, B.lo)
        d.ldb, d.strideB, d.b_entries = B.ld, B.stride, B.batch
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
    d.max_ctas = int(max_ctas)
    d.c_follows_d = 1 if c_follows_d else 0
    if A.f16 or B.f16:
        assert A.f16 and B.f16
        d.f16, d.kc = 1, CHAIN_K
        d.a_exp, d.b_exp, d.ab_exp0 = ip(A.exp), ip(B.exp), int(A.exp0 + B.exp0)
        d.out_exp, d.out_exp0, d.out_rel, d.out_exp_w = ip(out_exp), int(out_exp0), int(out_rel), ip(out_exp_w)
    if q is not None:
        d.q_code, d.q_in, d.q_absmax_in, d.q_diag_in = ip(q["code"]), ip(q["q_in"]), ip(q["absmax_in"]), ip(q["diag_in"])
        d.q_out, d.q_absmax_out, d.q_diag_out = ip(q["q_out"]), ip(q["absmax_out"]), ip(q["diag_out"])
        d.q_stride_codes, d.q_stride_absmax, d.q_stride_diag = q["stride_codes"], q["stride_absmax"], q["stride_diag"]
    with torch.cuda.device(A.hi.device):
        rc = F.lib.qt_gemm_ex(ct.byref(d), F._stream(A.hi))
    F._check(rc, f"gemm_ex ({b} x {M}x{N}x{K})")
