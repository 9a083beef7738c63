"""Batched execution of the preconditioner work of one optimizer step.

The reference walks parameters one by one and, inside, blocks and axes one by one
(optimizers/shampoo2.py:413-468, :169-272).  Here every preconditioner matrix of one
order lives in one contiguous arena (codes, scales, diagonals, spectra), and a step
processes a whole order class with batched launches: one dequantize, a few batched
products, one batched QR, one quantize.  The per-matrix arithmetic is the reference's:

  statistics refresh    shampoo2.py:169-200 + qtensor/utils.py:156-171, :192-203
  inverse 4th root      shampoo2.py:202-232 + qtensor/functional.py:749-762
                        (Schur-Newton: optimizers/matrix_functions.py:80-141)
  preconditioned grad   shampoo2.py:234-272
  dense variant         shampoo1.py:148-241
"""
import ctypes as ct
import math
from collections import defaultdict

import torch

import qtensor.functional as F
from optimizers import matrix_functions as MF
from optimizers._qr import householder_q
from optimizers import _gemm

_TEMP_ELEMS = 1 << 28          # cap on floats per batched temporary (1 GiB)

# The reference's low-bit dequantize_blockwise_diagreal returns None (it has no return
# statement, qtensor/functional.py:312-368), so its optimizers fall back to the identity
# preconditioner (shampoo2.py:255-261) and, in the dense flavour, re-seed the statistic with
# eps*I at every update (shampoo1.py:172-177, :187-197).  Setting this flag reproduces that
# behaviour so results can be compared with the unmodified reference; it is off by default.
REFERENCE_DIAGREAL_NONE = False


def _eps_identity(cls, m, eps):
    return (eps * torch.eye(cls.n, device=cls.device)).expand(m, -1, -1).clone()


def _ptr(t):
    return None if t is None else ct.c_void_p(t.data_ptr())


def _round_up(x, m):
    return (x + m - 1) // m * m


class QuantArena:
    """`count` square matrices of order n stored blockwise-quantized, contiguously.

    Low-bit layout per matrix: `row_bytes` packed code bytes (padded to 16), n*nb fp32
    scales and, for the diagreal flavour, n fp32 diagonal entries.  Orders whose n*n is
    below `min_lowbit_size`, and bit widths 16/32, are kept as plain matrices."""

    def __init__(self, n, count, device, bits, blocksize, code, min_lowbit_size, diagreal):
        self.n, self.count, self.device = n, count, device
        self.blocksize, self.code, self.diagreal = blocksize, code, diagreal
        self.lowbit = bits in (4, 8) and n * n >= min_lowbit_size
        self.bits = bits if self.lowbit else (16 if bits == 16 else 32)
        if self.lowbit:
            self.nb = (n + blocksize - 1) // blocksize
            self.nbytes = (n * n * bits + 7) // 8
            self.row_bytes = _round_up(self.nbytes, 16)
            self.var = torch.zeros(count, self.row_bytes, dtype=torch.uint8, device=device)
            self.absmax = torch.zeros(count, n * self.nb, dtype=torch.float32, device=device)
            self.diag = torch.zeros(count, n, dtype=torch.float32, device=device) if diagreal else None
        else:
            dt = torch.bfloat16 if self.bits == 16 else torch.float32
            self.var = torch.zeros(count, n, n, dtype=dt, device=device)
            self.absmax = self.diag = None

    def storage(self, i):
        if not self.lowbit:
            return {"var": self.var[i]}
        st = {"var": self.var[i, : self.nbytes], "absmax": self.absmax[i]}
        if self.diagreal:
            st["diag"] = self.diag[i]
        return st

    def copy_slot_from(self, other, dst, src):
        """Slot `dst` of this arena <- slot `src` of `other` (same order and format; any device)."""
        same = (self.n == other.n and self.lowbit == other.lowbit and self.bits == other.bits
                and self.diagreal == other.diagreal and (not self.lowbit or self.blocksize == other.blocksize))
        if not same:
            raise RuntimeError(f"quantized state of order {other.n} ({other.bits}-bit, block {other.blocksize}) cannot be "
                               f"loaded into state of order {self.n} ({self.bits}-bit, block {self.blocksize})")
        self.var[dst].copy_(other.var[src])
        if self.lowbit:
            self.absmax[dst].copy_(other.absmax[src])
            if self.diagreal:
                self.diag[dst].copy_(other.diag[src])

    def fusable(self):
        """True if a GEMM epilogue can read / write this arena's state directly
        (qt_gemm_bf16x3_q4 / x6_q4: 4-bit, block 64, order a multiple of 16, CUDA)."""
        return (self.lowbit and self.bits == 4 and self.blocksize == 64 and self.n % 16 == 0
                and self.var.is_cuda and USE_TENSOR_CORES and FUSE_STATE_EPILOGUE and F.lib is not None)

    def state(self, a, b):
        """(codes, absmax, diag or None) views of matrices a..b-1, the operand form of _gemm.matmul_q4."""
        return self.var[a:b], self.absmax[a:b], (self.diag[a:b] if self.diagreal else None)

    def operand(self, slots):
        """Matrices `slots` as a product operand that stays 4-bit: dequantized tile by tile inside
        the product kernel (no fp32 copy, no operand planes in device memory)."""
        idx = _index_tensor(list(slots), self.device, torch.int32)
        return _gemm.StateOperand(self.var, self.absmax, self.diag if self.diagreal else None, self.code, self.n, idx)

    def dequantize_planes(self, slots):
        """Matrices `slots` (any order, repeats allowed) as bf16 hi/lo Planes, written by the
        dequantize kernel itself: no fp32 copy, no gather, no split pass (qt_dequantize_planes)."""
        n, m = self.n, len(slots)
        idx = _index_tensor(list(slots), self.device, torch.int32)
        if _gemm.FP16_PLANES:
            scratch = torch.empty(2, m, dtype=torch.int32, device=self.device)     # amax bits, exponents
            P = _gemm.Planes(m, n, n, self.device, f16=True, exp=scratch[1], tmax=_gemm.SPLIT_TARGET)
            with torch.cuda.device(self.device):
                rc = F.lib.qt_dequantize_planes_f16(
                    _ptr(self.var), self.row_bytes, _ptr(self.code), n, m, _ptr(self.absmax), n * self.nb,
                    _ptr(self.diag) if self.diagreal else None, n, _ptr(idx), _ptr(scratch[0]), _gemm.SPLIT_TARGET,
                    _ptr(scratch[1]), P.ptr_hi(), P.ptr_lo(), P.ld, P.stride, self.blocksize, self.bits, F._stream(self.var))
            F._check(rc, "dequantize to planes")
            return P
        P = _gemm.Planes(m, n, n, self.device)
        with torch.cuda.device(self.device):
            rc = F.lib.qt_dequantize_planes(
                _ptr(self.var), self.row_bytes, _ptr(self.code), n, m, _ptr(self.absmax), n * self.nb,
                _ptr(self.diag) if self.diagreal else None, n, _ptr(idx),
                P.ptr_hi(), P.ptr_lo(), P.ld, P.stride, self.blocksize, self.bits, F._stream(self.var))
        F._check(rc, "dequantize to planes")
        return P

    def dequantize(self, a, b):
        """fp32 (b-a, n, n) copy of matrices a..b-1."""
        if not self.lowbit:
            return self.var[a:b].float().clone()
        n, m = self.n, b - a
        out = torch.empty(m, n, n, dtype=torch.float32, device=self.device)
        F._require_lib(self.var)
        with torch.cuda.device(self.device):
            rc = F.lib.qt_dequantize_blockwise(
                _ptr(self.var[a:b]), self.row_bytes, _ptr(self.code), n, m,
                _ptr(self.absmax[a:b]), n * self.nb,
                _ptr(self.diag[a:b]) if self.diagreal else None, n,
                _ptr(out), 0, n * n, self.blocksize, self.bits, F._stream(self.var))
        F._check(rc, "batched dequantize")
        return out

    def quantize(self, a, b, X):
        """Store the fp32 batch X (b-a, n, n), contiguous."""
        if not self.lowbit:
            self.var[a:b].copy_(X)
            return
        n, m = self.n, b - a
        X = X.contiguous()
        assert X.shape == (m, n, n) and X.dtype == torch.float32
        with torch.cuda.device(self.device):
            rc = F.lib.qt_quantize_blockwise(
                _ptr(X), 0, n * n, _ptr(self.code), n, m,
                _ptr(self.absmax[a:b]), n * self.nb,
                _ptr(self.diag[a:b]) if self.diagreal else None, n,
                _ptr(self.var[a:b]), self.row_bytes, self.blocksize, self.bits, F._stream(self.var))
        F._check(rc, "batched quantize")


class OrderClass:
    """State arenas of every preconditioner matrix of order n owned by one parameter group."""

    def __init__(self, n, count, device, flavour, bits, blocksize, code, min_lowbit_size, rect_t1, rect_t2):
        self.n, self.count, self.device, self.flavour = n, count, device, flavour
        self.rect_t1, self.rect_t2 = rect_t1, rect_t2
        self.keep = max(1, n // 2)
        self.stat = QuantArena(n, count, device, bits, blocksize, code, min_lowbit_size, diagreal=(flavour == "s1"))
        self.prec = QuantArena(n, count, device, bits, blocksize, code, min_lowbit_size, diagreal=True)
        if flavour == "s2":
            self.S = torch.zeros(count, self.keep, dtype=torch.float32, device=device)
            self.keep_idx = torch.zeros(count, self.keep, dtype=torch.int64, device=device)
            self.max_eig = torch.zeros(count, dtype=torch.float32, device=device)
        self._next = 0

    def alloc(self):
        i = self._next
        assert i < self.count
        self._next += 1
        return i

    def stat_storage(self, i):
        st = self.stat.storage(i)
        if self.flavour == "s2":
            st.update(Svalue=self.S[i], keep_indices=self.keep_idx[i], max_eigenvalue=self.max_eig[i])
        return st

    def sub_batch(self):
        return max(1, _TEMP_ELEMS // (self.n * self.n))

    def copy_slot_from(self, other, dst, src):
        """Everything slot `src` of `other` holds (statistic, spectrum, preconditioner) into slot `dst`."""
        if self.flavour != other.flavour:
            raise RuntimeError(f"checkpoint holds '{other.flavour}' statistics, this optimizer keeps '{self.flavour}'")
        self.stat.copy_slot_from(other.stat, dst, src)
        self.prec.copy_slot_from(other.prec, dst, src)
        if self.flavour == "s2":
            self.S[dst].copy_(other.S[src])
            self.keep_idx[dst].copy_(other.keep_idx[src])
            self.max_eig[dst].copy_(other.max_eig[src])


# ---------------------------------------------------------------------------------------
# The dense products of the hot path, one named operation each.
#
# On CUDA they run on the library's tcgen05 kernel (optimizers/_gemm.py): operands are
# carried as bf16 hi/lo planes, a product chain hands planes from one epilogue to the next
# prologue, and transposes are operand-major flags, not copies.  On CPU tensors (32-bit
# state, used by the host-logic tests) the same operations are plain torch products.
# ---------------------------------------------------------------------------------------
USE_TENSOR_CORES = True
FUSE_STATE_EPILOGUE = True     # products that end in 4-bit state quantize inside the GEMM epilogue
DEQUANTIZE_TO_PLANES = True    # preconditioners are dequantized straight into operand planes, never to fp32
# ... or inside the product itself (converter warps of the product kernel).  A tile of the 4-bit
# operand is converted once per output tile that uses it, so this pays while few output tiles share
# an operand tile (measured on the ViT-B/32 apply products, where 6 to 24 column tiles share each
# tile of P: 5.9 ms per steady-state step against 4.1 ms through planes written once); with
# DEQUANTIZE_IN_PRODUCT_MAX_SHARE = None every eligible product takes this path.
DEQUANTIZE_IN_PRODUCT = True
DEQUANTIZE_IN_PRODUCT_MAX_SHARE = 2
# Set while an order class with plain 16/32-bit state, or a Schur-Newton inverse root, is
# processed: those paths have no quantisation noise to hide the ~1e-5 relative error of the
# split-bf16 products (and the Newton iteration amplifies it), so they stay on fp32 products.
_EXACT = False


class _exact:
    def __init__(self, on):
        self.on = on

    def __enter__(self):
        global _EXACT
        self.prev, _EXACT = _EXACT, (_EXACT or self.on)

    def __exit__(self, *exc):
        global _EXACT
        _EXACT = self.prev


class Mat:
    """A batch of matrices available as an fp32 tensor, as operand planes, or both.  `bound`: an
    a-priori bound on the entries (float, or per-matrix fp32 tensor) that spares the split its pass
    for the largest magnitude; a violated bound trips QT_ERR_RANGE instead of passing silently."""

    def __init__(self, f32=None, planes=None, bound=None):
        self.f32, self._planes, self.bound = f32, planes, bound

    @property
    def planes3(self):
        if getattr(self, "_planes3", None) is None:
            x = self.f32 if self.f32.stride(2) == 1 else self.f32.contiguous()
            self._planes3 = _gemm.split3(x)
        return self._planes3

    @property
    def planes(self):
        if self._planes is None:
            x = self.f32 if self.f32.stride(2) == 1 else self.f32.contiguous()
            self._planes = _gemm.split(x, bound=self.bound)
        return self._planes


def _tc(t):
    return USE_TENSOR_CORES and not _EXACT and t.is_cuda and F.lib is not None


def mm(A, B, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, C=None, want_float=True, want_planes=False,
       out_bound=None):
    """alpha * op(A) @ op(B) + beta * C over a batch; A, B are Mat, C an fp32 tensor.  On CUDA the
    product runs on the tensor cores from scaled fp16 planes (fp32-level accuracy).  `out_bound`:
    a-priori bound on |result| used to place a plane output (see _gemm.matmul)."""
    ref = A.f32 if A.f32 is not None else A._planes.hi
    if _tc(ref):
        D, P = _gemm.matmul(A.planes, B.planes, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta, C=C,
                            want_float=want_float, want_planes=want_planes, out_bound=out_bound)
        return Mat(D, P)
    a = A.f32.transpose(1, 2) if trans_a else A.f32
    b = B.f32.transpose(1, 2) if trans_b else B.f32
    if C is not None and beta != 0.0:
        return Mat(torch.baddbmm(C, a, b, beta=beta, alpha=alpha))
    out = torch.bmm(a, b)
    return Mat(out if alpha == 1.0 else out * alpha)


# Entries of a (nearly) orthonormal basis and of its Gram matrix stay below these bounds with a
# wide margin (rows of a 4-bit eigenbasis have norm 1 +- 0.2); a plane output placed with them
# keeps 22 significant bits.  An input that violates them trips QT_ERR_RANGE instead of passing
# silently.
_BASIS_BOUND = 8.0
_GRAM_BOUND = 16.0
_UNIT_BOUND = 2.0             # entries of orthonormal rows / columns and of Householder vectors (<= 1) with margin


def op_bjorck(V, want_planes=False):
    """1.5 V - 0.5 (V V^T) V on the rows of each V in the batch (utils.py:196, functional.py:757)."""
    tc = _tc(V.f32)
    W = mm(V, V, trans_b=True, want_float=not tc, want_planes=tc, out_bound=_GRAM_BOUND)
    return mm(W, V, alpha=-0.5, beta=1.5, C=V.f32, want_planes=want_planes and tc, out_bound=_BASIS_BOUND)


def op_scaled_gram(rows, weights, want_planes=False):
    """rows^T diag(weights) rows (utils.py:203, functional.py:762)."""
    scaled = Mat(weights.unsqueeze(2) * rows.f32)
    return mm(rows, scaled, trans_a=True, want_planes=want_planes and _tc(rows.f32))


def op_scaled_gram_gathered(Vt, idx, weights):
    """rows^T diag(weights) rows with rows = Vt[idx] (utils.py:202-203); Vt fp32 (b, n, n), idx int64
    (b, k), weights fp32 (b, k).  On the tensor-core path the gather and the scaling happen while
    the operands are split into planes, so neither rows nor the scaled copy is materialised."""
    if _tc(Vt) and Vt.stride(2) == 1:
        A = _gemm.split_rows(Vt, idx, bound=_BASIS_BOUND)
        B = _gemm.split_rows(Vt, idx, weights.contiguous(), bound=(weights.abs().amax(dim=1) * _BASIS_BOUND).contiguous())
        D, _ = _gemm.matmul(A, B, trans_a=True)
        return Mat(D)
    return op_scaled_gram(Mat(_gather_rows(Vt, idx)), weights)


def op_ema_gram(L, G, axis, w1, w2):
    """w1 L + w2 G G^T (axis 0) or w1 L + w2 G^T G (axis 1) (shampoo2.py:185-199); L fp32 tensor.

    The statistic's small eigenvalues (the half of the spectrum that is kept, regularised by only
    matrix_eps * lambda_max) must be accurate to ~1e-7 * lambda_max: this needs the 22-bit operand
    planes and the short accumulation chains of the fp16-plane product."""
    Gm = Mat(G)
    if axis == 0:
        return mm(Gm, Gm, trans_b=True, alpha=w2, beta=w1, C=L).f32
    return mm(Gm, Gm, trans_a=True, alpha=w2, beta=w1, C=L).f32


def op_ema_gram_selected(L, sel, G, axis, w1, w2):
    """op_ema_gram on the matrices L[sel[k]] with G[k], updated in place: the product reads its C
    operand and writes its result through the slot list, so the selected matrices are neither
    gathered into a temporary nor scattered back (sel: int32 device tensor)."""
    P = Mat(G).planes
    _gemm.gemm_ex(P, P, trans_a=(axis == 1), trans_b=(axis == 0), alpha=w2, beta=w1, C=L, D=L,
                  d_slot=sel, c_follows_d=True, batch=G.shape[0])
    return L


def op_subspace_step(L, Vt):
    """Orthonormal basis of L V (one subspace-iteration step, utils.py:157) and the Rayleigh
    quotients diag(V^T L V) (utils.py:158).  L, Vt are Mat; returns fp32 tensors."""
    V, Vp = householder_q(mm(L, Vt, trans_b=True).f32, tensor_cores=_tc(L.f32), with_planes=True)
    LV = mm(L, Mat(V, planes=Vp, bound=_UNIT_BOUND)).f32            # the QR hands over the planes it kept of Q
    return V, column_dot(LV, V)


def column_dot(A, B):
    """out[b, j] = sum_i A[b, i, j] B[b, i, j] with an order of summation that depends on the matrix
    shape only (qt_column_dot); plain torch off CUDA."""
    if not (A.is_cuda and F.lib is not None and A.dtype == torch.float32 and B.dtype == torch.float32):
        return (A * B).sum(dim=1)
    A, B = A.contiguous(), B.contiguous()
    b, r, c = A.shape
    out = torch.empty(b, c, dtype=torch.float32, device=A.device)
    with torch.cuda.device(A.device):
        rc = F.lib.qt_column_dot(ct.c_void_p(A.data_ptr()), ct.c_void_p(B.data_ptr()), c, r * c, r, c, b,
                                 ct.c_void_p(out.data_ptr()), c, F._stream(A))
    F._check(rc, "column_dot")
    return out


def op_apply(P0, G, P1):
    """P0 G P1 (shampoo2.py:265-268); fp32 tensors in and out."""
    T = mm(Mat(P0), Mat(G), want_float=not _tc(G), want_planes=_tc(G))
    return mm(T, Mat(P1)).f32


def _runs(indices):
    """Sorted slot numbers -> list of (a, b, positions) with contiguous slots a..b-1."""
    order = sorted(range(len(indices)), key=lambda k: indices[k])
    out, start = [], 0
    for j in range(1, len(order) + 1):
        if j == len(order) or indices[order[j]] != indices[order[j - 1]] + 1:
            a = indices[order[start]]
            out.append((a, indices[order[j - 1]] + 1, order[start:j]))
            start = j
    return out


def _split_runs(runs, cap):
    for a, b, pos in runs:
        for s in range(a, b, cap):
            e = min(b, s + cap)
            yield s, e, pos[s - a: e - a]


def _gather_rows(Vt, idx):
    n = Vt.shape[2]
    return torch.gather(Vt, 1, idx.unsqueeze(2).expand(-1, -1, n))


_INDEX_CACHE = {}


def _index_tensor(ks, device, dtype=torch.int64):
    """Device copy of a small index list, cached: the same lists recur every step, and a
    host-to-device copy is not allowed while a CUDA graph is being captured."""
    key = (str(device), tuple(ks), dtype)
    t = _INDEX_CACHE.get(key)
    if t is None:
        t = _INDEX_CACHE[key] = torch.tensor(ks, device=device, dtype=dtype)
    return t


def _ema_update_fused(arena, a, grads_axes, w1, w2):
    """state[a+k] <- quantize(w1 dequantize(state[a+k]) + w2 (G_k G_k^T | G_k^T G_k)) with the state read and
    written by the product's epilogue (no fp32 copy of L).  Needs every group of equally shaped
    blocks to occupy consecutive slots; returns False (nothing done) otherwise."""
    groups = defaultdict(list)
    for k, (g, axis) in enumerate(grads_axes):
        groups[(tuple(g.shape), axis)].append(k)
    if any(ks != list(range(ks[0], ks[0] + len(ks))) for ks in groups.values()):
        return False
    for (shape, axis), ks in groups.items():
        P = _gemm.split(torch.stack([grads_axes[k][0].float() for k in ks]))
        st = arena.state(a + ks[0], a + ks[0] + len(ks))
        _gemm.matmul_q4(P, P, arena.code, st, trans_a=(axis == 1), trans_b=(axis == 0), alpha=w2, beta=w1, old=st)
    return True


def _ema_update(L, grads_axes, w1, w2):
    """L[k] <- w1 L[k] + w2 * (G_k G_k^T | G_k^T G_k); blocks of equal shape are stacked."""
    groups = defaultdict(list)
    for k, (g, axis) in enumerate(grads_axes):
        groups[(tuple(g.shape), axis)].append(k)
    for (shape, axis), ks in groups.items():
        Gs = torch.stack([grads_axes[k][0].float() for k in ks])
        if len(ks) == L.shape[0]:
            L = op_ema_gram(L, Gs, axis, w1, w2)
        elif _tc(L) and L.is_contiguous():
            L = op_ema_gram_selected(L, _index_tensor(ks, L.device, torch.int32), Gs, axis, w1, w2)
        else:
            sel = _index_tensor(ks, L.device)
            L[sel] = op_ema_gram(L[sel], Gs, axis, w1, w2)
    return L


PARALLEL_CLASSES = True        # order classes are independent: run them on separate CUDA streams
_STREAMS = {}
_NUM_STREAMS = 8


def _over_classes(by_class, payload=None):
    """Yields (cls, payload) for every order class; on CUDA each class is issued on one of a few
    side streams so that the latency-bound work of small classes (a QR of 12 matrices is 35
    sequential panel steps) overlaps with the other classes.  Joined back before returning."""
    classes = sorted(by_class.items(), key=lambda kv: -(kv[0].n ** 3) * len(kv[1]))
    dev = classes[0][0].device if classes else None
    if payload is not None:
        classes = [(cls, payload[cls]) for cls, _ in classes]
    if not PARALLEL_CLASSES or len(classes) < 2 or dev is None or torch.device(dev).type != "cuda":
        for cls, item in classes:
            yield cls, item
        return
    pool = _STREAMS.get(str(dev))
    if pool is None:
        pool = _STREAMS[str(dev)] = [torch.cuda.Stream(device=dev) for _ in range(_NUM_STREAMS)]
    main = torch.cuda.current_stream(dev)
    used = pool[: min(len(pool), len(classes))]
    for s in used:
        s.wait_stream(main)
    for i, (cls, item) in enumerate(classes):
        with torch.cuda.stream(used[i % len(used)]):
            yield cls, item
    for s in used:
        main.wait_stream(s)


SPLIT_CLASSES = False          # cut a class that dominates the step into slot ranges on separate streams (more,
                               # smaller launches).  Off: with today's kernels whole classes are faster at every shard
                               # size (ViT-B/32 step 30.3 vs 31.5 ms on one GPU, 16.5 vs 16.8 for half, 7.0 vs 7.1 for an eighth)
_UNIT_TARGET = 6               # aim for about this many equally expensive units per refresh


def _split_units(merged):
    """{cls: (stat entries, root slots)} -> list of (cost, cls, (entries, slots)) work units.

    The step's critical path is the largest class: its chain of latency-bound launches (a QR of
    62 order-1200 matrices is ~40 panel launches that each occupy 62 SMs) runs on one stream while
    the small classes finish early.  Cutting such a class into contiguous slot ranges lets those
    chains run side by side; a slot's statistics and inverse root stay in the same unit."""
    cost = {cls: float(cls.n) ** 3 * len(set([e[0] for e in v[0]] + list(v[1]))) for cls, v in merged.items()}
    total = sum(cost.values())
    units = []
    for cls, (entries, slots) in merged.items():
        parts = 1
        if SPLIT_CLASSES and total > 0 and torch.device(cls.device).type == "cuda":
            parts = max(1, min(4, int(round(cost[cls] / (total / _UNIT_TARGET)))))
        ids = sorted(set([e[0] for e in entries] + list(slots)))
        parts = min(parts, max(1, len(ids) // 8))          # keep at least 8 matrices per unit
        if parts == 1:
            units.append((cost[cls], cls, (entries, slots)))
            continue
        step = (len(ids) + parts - 1) // parts
        for k in range(parts):
            chunk = set(ids[k * step: (k + 1) * step])
            if chunk:
                units.append((cost[cls] * len(chunk) / len(ids), cls,
                              ([e for e in entries if e[0] in chunk], [x for x in slots if x in chunk])))
    return units


def _over_units(units):
    """Yields (cls, item) for every (cost, cls, item) unit, most expensive first, each on one of a
    few side streams on CUDA; joined back before returning."""
    units = sorted(units, key=lambda u: -u[0])
    dev = units[0][1].device if units else None
    if not PARALLEL_CLASSES or len(units) < 2 or dev is None or torch.device(dev).type != "cuda":
        for _, cls, item in units:
            yield cls, item
        return
    pool = _STREAMS.get(str(dev))
    if pool is None:
        pool = _STREAMS[str(dev)] = [torch.cuda.Stream(device=dev) for _ in range(_NUM_STREAMS)]
    main = torch.cuda.current_stream(dev)
    used = pool[: min(len(pool), len(units))]
    for st in used:
        st.wait_stream(main)
    for i, (_, cls, item) in enumerate(units):
        with torch.cuda.stream(used[i % len(used)]):
            yield cls, item
    for st in used:
        main.wait_stream(st)


def add_statistics(items, w1, w2, eps=1e-6, exact=False):
    """items: list of (OrderClass, slot, grad_block, axis).  Refreshes the statistics.
    `exact` keeps every product in fp32 (used when the inverse root is the Schur-Newton
    iteration, which amplifies operand rounding)."""
    by_class = defaultdict(list)
    for cls, slot, g, axis in items:
        by_class[cls].append((slot, g, axis))
    for cls, entries in _over_classes(by_class):
        _class_statistics(cls, entries, w1, w2, eps, exact)


def _class_statistics(cls, entries, w1, w2, eps, exact):
        runs = _runs([e[0] for e in entries])
        for a, b, pos in _split_runs(runs, cls.sub_batch()):
          # the dense flavour re-quantises L itself and then runs the Newton iteration on it:
          # a 1e-5 operand error flips a few 4-bit codes and the iteration amplifies them
          with _exact(exact or not cls.stat.lowbit or cls.flavour == "s1"):
            ga = [(entries[p][1], entries[p][2]) for p in pos]
            if cls.flavour == "s1":
                if REFERENCE_DIAGREAL_NONE and cls.stat.lowbit:
                    L = _eps_identity(cls, b - a, eps)
                elif cls.stat.fusable() and not exact and _ema_update_fused(cls.stat, a, ga, w1, w2):
                    continue
                else:
                    L = cls.stat.dequantize(a, b)
                cls.stat.quantize(a, b, _ema_update(L, ga, w1, w2))
                continue
            Vt = Mat(cls.stat.dequantize(a, b), bound=_UNIT_BOUND if cls.stat.lowbit else None)
            if cls.stat.lowbit:
                for _ in range(cls.rect_t1):
                    Vt = op_bjorck(Vt, want_planes=True)
            L = op_scaled_gram_gathered(Vt.f32, cls.keep_idx[a:b], cls.S[a:b]).f32
            L = _ema_update(L, ga, w1, w2)
            V, eigs = op_subspace_step(Mat(L), Vt)
            vals, idx = torch.sort(eigs, dim=1)
            cls.keep_idx[a:b] = idx[:, : cls.keep]
            cls.S[a:b] = vals[:, : cls.keep]
            cls.max_eig[a:b] = eigs.amax(dim=1)
            cls.stat.quantize(a, b, V.transpose(1, 2).contiguous())


def _newton_starts(root_items, inv_root_mode):
    """Start vectors of the power iterations behind the Schur-Newton roots, drawn one matrix at
    a time in the order the reference reaches them (parameter by parameter, statistic by
    statistic: shampoo2.py:206-230 -> matrix_functions.py:36), whatever order the classes are
    processed in afterwards.  {(class, slot): vector}; empty when no class takes the Newton path."""
    starts = {}
    for cls, slot in root_items:
        if (cls.flavour == "s1" or inv_root_mode != 0) and cls.n >= 2:
            starts[(cls, slot)] = MF.draw_start_vectors(1, cls.n, cls.device)[0]
    return starts


def compute_preconditioners(items, eps, inv_root_mode, exponent=4):
    """items: list of (OrderClass, slot).  Writes L^(-1/exponent) into the preconditioner arenas."""
    starts = _newton_starts(items, inv_root_mode)
    by_class = defaultdict(list)
    for cls, slot in items:
        by_class[cls].append(slot)
    for cls, slots in _over_classes(by_class):
        _class_roots(cls, slots, eps, inv_root_mode, exponent, starts)


def refresh(stat_items, root_items, w1, w2, eps, inv_root_mode, exact=False, exponent=4):
    """add_statistics followed by compute_preconditioners, pipelined per order class: a class
    starts its inverse roots as soon as its own statistics are done, on the same stream."""
    starts = _newton_starts(root_items, inv_root_mode)
    stats, roots = defaultdict(list), defaultdict(list)
    for cls, slot, g, axis in stat_items:
        stats[cls].append((slot, g, axis))
    for cls, slot in root_items:
        roots[cls].append(slot)
    merged = {cls: (stats.get(cls, []), roots.get(cls, [])) for cls in list(stats) + [c for c in roots if c not in stats]}
    for cls, (entries, slots) in _over_units(_split_units(merged)):
        if entries:
            _class_statistics(cls, entries, w1, w2, eps, exact)
        if slots:
            _class_roots(cls, slots, eps, inv_root_mode, exponent, starts)


def _class_roots(cls, slots, eps, inv_root_mode, exponent, starts=None):
        def v0_of(a, b):
            if not starts:
                return None
            return torch.stack([starts[(cls, s)] for s in range(a, b)])
        for a, b, _ in _split_runs(_runs(slots), cls.sub_batch()):
          with _exact((not cls.stat.lowbit) or cls.flavour == "s1" or inv_root_mode != 0):
            if cls.flavour == "s1":
                if REFERENCE_DIAGREAL_NONE and cls.stat.lowbit:
                    L = _eps_identity(cls, b - a, eps)
                else:
                    L = cls.stat.dequantize(a, b)
                P = MF.ComputePower(L, exponent, ridge_epsilon=eps, v0=v0_of(a, b))
            elif inv_root_mode == 0:
                Vt = cls.stat.dequantize(a, b)
                rows = Mat(_gather_rows(Vt, cls.keep_idx[a:b]), bound=_UNIT_BOUND if cls.stat.lowbit else None)
                if cls.stat.lowbit:
                    for _ in range(cls.rect_t2):
                        rows = op_bjorck(rows, want_planes=True)
                rho = eps * cls.max_eig[a:b]
                weights = F.ridged_inverse_root(cls.S[a:b], rho.unsqueeze(1), exponent)
                if cls.prec.fusable() and _tc(rows.f32 if rows.f32 is not None else rows._planes.hi):
                    # rows^T diag(w) rows straight into the 4-bit preconditioner (quantized in the epilogue)
                    scaled = _gemm.split_rows(rows.f32, None, weights.contiguous(),
                                              bound=(weights.abs().amax(dim=1) * _BASIS_BOUND).contiguous())
                    _gemm.matmul_q4(rows.planes, scaled, cls.prec.code, cls.prec.state(a, b), trans_a=True)
                    continue
                P = op_scaled_gram(rows, weights).f32
            else:
                Vt = Mat(cls.stat.dequantize(a, b))
                if cls.stat.lowbit:
                    for _ in range(cls.rect_t1):
                        Vt = op_bjorck(Vt)
                rows = Mat(_gather_rows(Vt.f32, cls.keep_idx[a:b]))
                P = MF.ComputePower(op_scaled_gram(rows, cls.S[a:b]).f32.contiguous(), exponent, ridge_epsilon=eps, v0=v0_of(a, b))
            cls.prec.quantize(a, b, P)


def _planes_direct(cls, dtype):
    """True if this class's preconditioners can be dequantized straight into product operands."""
    a = cls.prec
    return (a.lowbit and a.n % 8 == 0 and dtype == torch.float32 and a.var.is_cuda and USE_TENSOR_CORES
            and DEQUANTIZE_TO_PLANES and F.lib is not None and not _EXACT and not REFERENCE_DIAGREAL_NONE)


def preconditioned_blocks(items):
    """items: list of (cls0, slot0, cls1, slot1, grad_block).  Returns [P0 G P1 for each]."""
    out = [None] * len(items)
    # Fast path: 4-bit preconditioners are only ever product operands here, so they are dequantized
    # straight into bf16 planes, already stacked in the order of the blocks that use them.
    rest = []
    direct = defaultdict(list)
    for k, (c0, s0, c1, s1, g) in enumerate(items):
        if _planes_direct(c0, g.dtype) and _planes_direct(c1, g.dtype):
            direct[(c0, c1, tuple(g.shape))].append(k)
        else:
            rest.append(k)
    for (c0, c1, shape), ks in direct.items():
        cap = max(1, _TEMP_ELEMS // max(shape[0] * shape[0], shape[1] * shape[1], 1))
        for s in range(0, len(ks), cap):
            part = ks[s: s + cap]
            G = torch.stack([items[k][4] for k in part])
            def operand(c, sl, sharing_tiles):
                ok = (DEQUANTIZE_IN_PRODUCT and _gemm.FP16_PLANES and c.prec.bits == 4 and c.prec.blocksize == 64 and c.n % 16 == 0
                      and (DEQUANTIZE_IN_PRODUCT_MAX_SHARE is None or sharing_tiles <= DEQUANTIZE_IN_PRODUCT_MAX_SHARE))
                return c.prec.operand(sl) if ok else c.prec.dequantize_planes(sl)
            # P0 (m x m) is the left operand of P0 G: each of its tiles serves ceil(k / 128) output tiles;
            # P1 (k x k) is the right operand of (P0 G) P1: each tile serves ceil(m / 128) output tiles
            P0 = Mat(planes=operand(c0, [items[k][1] for k in part], (shape[1] + 127) // 128))
            P1 = Mat(planes=operand(c1, [items[k][3] for k in part], (shape[0] + 127) // 128))
            T = mm(P0, Mat(G), want_float=False, want_planes=True)
            R = mm(T, P1).f32
            for j, k in enumerate(part):
                out[k] = R[j]
    if not rest:
        return out
    for k, r in zip(rest, _preconditioned_blocks_general([items[k] for k in rest])):
        out[k] = r
    return out


def _preconditioned_blocks_general(items):
    needed = defaultdict(set)
    for c0, s0, c1, s1, _ in items:
        needed[c0].add(s0)
        needed[c1].add(s1)
    cache = {}
    for cls, slots in needed.items():
        for a, b, _ in _split_runs(_runs(sorted(slots)), cls.sub_batch()):
            if REFERENCE_DIAGREAL_NONE and cls.prec.lowbit:
                P = _eps_identity(cls, b - a, 1.0)
            else:
                P = cls.prec.dequantize(a, b)
            for s in range(a, b):
                cache[(cls, s)] = P[s - a]
    out = [None] * len(items)
    groups = defaultdict(list)
    for k, (c0, s0, c1, s1, g) in enumerate(items):
        groups[tuple(g.shape)].append(k)
    for shape, ks in groups.items():
        cap = max(1, _TEMP_ELEMS // max(shape[0] * shape[0], shape[1] * shape[1], 1))
        for s in range(0, len(ks), cap):
            part = ks[s: s + cap]
            dt = items[part[0]][4].dtype
            G = torch.stack([items[k][4] for k in part])
            P0 = torch.stack([cache[(items[k][0], items[k][1])] for k in part]).to(dt)
            P1 = torch.stack([cache[(items[k][2], items[k][3])] for k in part]).to(dt)
            lowbit = items[part[0]][0].prec.lowbit and items[part[0]][2].prec.lowbit and dt == torch.float32
            with _exact(not lowbit):
                R = op_apply(P0, G, P1)
            for j, k in enumerate(part):
                out[k] = R[j]
    return out
