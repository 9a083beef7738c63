"""Batched Householder QR (Q factor only) for a stack of square matrices.

Replaces the per-matrix torch.linalg.qr of the reference's eigenbasis refresh
(qtensor/utils.py:157).  Blocked compact-WY algorithm with 32-column panels: the panel
factorisation of every matrix of the batch is one launch of the library's
qt_householder_panel kernel; the trailing update  A <- (I - V T^T V^T) A  and the backward
accumulation  Q <- (I - V T V^T) Q  are batched products.  Sign conventions are LAPACK's,
so Q agrees with torch.linalg.qr's up to rounding on full-rank input.
"""
import ctypes as ct
import warnings

import torch

import qtensor.functional as F

PANEL = 32
MAX_ORDER = 1216            # the panel kernel keeps a (rows x 32) panel in registers, 38 rows per lane


def _ptr(t):
    return ct.c_void_p(t.data_ptr())


OUTER = 128                 # columns per outer block (four panels): trailing updates are rank-128
USE_TENSOR_CORES = True     # rank-128 far updates on the tcgen05 kernel (rank-32 ones inside a block: fused into the panel kernel)


def _reflect(Vk, Tk, target, target_planes, transpose_t, Pv=None, Pt=None):
    """target <- (I - Vk T' Vk^T) target with T' = T^T (transpose_t) or T, fp32 in place.
    With `target_planes` (the operand planes of `target`) everything runs on the tensor cores:
    Y = Vk T' and W = Vk^T target are produced directly as operand planes, then
    target <- target - Y W with the planes of `target` kept in step.  `Pv`, `Pt`: planes of Vk, Tk."""
    from optimizers import _gemm
    if target_planes is None:
        W = torch.bmm(Vk.transpose(1, 2), target)
        W = torch.bmm(Tk.transpose(1, 2) if transpose_t else Tk, W)
        target.baddbmm_(Vk, W, alpha=-1.0)
        return
    if Pv is None:
        Pv = _gemm.split(Vk, bound=2.0)
    if Pt is None:
        Pt = _gemm.split(Tk)
    _, Yp = _gemm.matmul(Pv, Pt, trans_b=transpose_t, want_float=False, want_planes=True)
    _, Wp = _gemm.matmul(Pv, target_planes, trans_a=True, want_float=False, want_planes=True)
    _gemm.matmul(Yp, Wp, alpha=-1.0, beta=1.0, C=target, out=target, out_planes=target_planes)


def _merge_t(Vo, Tp, widths, Pv=None):
    """Triangular factor of a block of panels: H_1 .. H_p = I - Vo T Vo^T from the panels' own
    factors Tp[k] (LAPACK larft recurrence on blocks): T[:c, c:c+w] = -T[:c, :c] (Vo[:, :c]^T Vo[:, c:c+w]) Tk.
    With `Pv` (planes of Vo) the Gram matrix Vo^T Vo is a tensor-core product."""
    B = Vo.shape[0]
    wo = sum(widths)
    if Pv is not None and len(widths) > 1 and wo <= 128 and Tp.stride(3) == 1 and Tp.stride(2) == PANEL and Tp.stride(1) == PANEL * PANEL:
        # one launch: Gram matrix on the tensor cores, recurrence in the library's merge kernel
        from optimizers import _gemm
        G, _ = _gemm.matmul(Pv, Pv, trans_a=True)
        T = torch.empty(B, wo, wo, dtype=torch.float32, device=Vo.device)
        with torch.cuda.device(Vo.device):
            rc = F.lib.qt_merge_t(_ptr(G), G.stride(1), G.stride(0), _ptr(Tp), Tp.stride(0), wo, B,
                                  _ptr(T), wo * wo, F._stream(Vo))
        F._check(rc, "merge_t")
        return T
    T = torch.zeros(B, wo, wo, dtype=torch.float32, device=Vo.device)
    G = None
    if len(widths) > 1:
        if Pv is not None:
            from optimizers import _gemm
            G, _ = _gemm.matmul(Pv, Pv, trans_a=True)
        else:
            G = torch.bmm(Vo.transpose(1, 2), Vo)
    c = 0
    for k, w in enumerate(widths):
        Tk = Tp[:, k, :w, :w]
        T[:, c:c + w, c:c + w] = Tk
        if c:
            T[:, :c, c:c + w] = -torch.bmm(torch.bmm(T[:, :c, :c], G[:, :c, c:c + w]), Tk)
        c += w
    return T


LOOKAHEAD = False           # far update split into the next block's columns (critical path) and the rest (side stream);
                            # measured: 5 % faster for 8 matrices of order 1200, 5-15 % slower from 16 matrices up - off
FORWARD_Q = True            # Q accumulated block by block beside the factorisation (with LOOKAHEAD), else backwards afterwards

_SIDE_STREAMS = {}
_WARNED_LARGE = False


def _side_streams(device):
    """Two side streams per (device, calling stream): order classes factor concurrently on
    streams of their own, and each of them needs its own pair."""
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    pair = _SIDE_STREAMS.get(key)
    if pair is None:
        pair = _SIDE_STREAMS[key] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
    return pair


def _apply_block(Yp, Pv, target, target_planes, max_ctas=0):
    """target <- target - Y (V^T target), fp32 and planes in one epilogue.  `max_ctas`: see
    _background_ctas()."""
    from optimizers import _gemm
    _, Wp = _gemm.matmul(Pv, target_planes, trans_a=True, want_float=False, want_planes=True, max_ctas=max_ctas)
    _gemm.matmul(Yp, Wp, alpha=-1.0, beta=1.0, C=target, out=target, out_planes=target_planes, max_ctas=max_ctas)
    return Wp


def _background_ctas(device, batch):
    """CTA cap of the products issued on the side streams.  The product kernel is persistent: it
    takes every SM until it is done, and a panel launch (one CTA per matrix, the critical path)
    issued meanwhile would wait for the whole product.  The cap leaves the panel kernel its SMs.
    0: no room for background work."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    free = sms - batch - 4
    return free if free >= sms // 4 else 0


def householder_q(X, tensor_cores=True, with_planes=False):
    """Q of the QR factorisation of each X[b] (X: (B, n, n) fp32 CUDA, overwritten).
    `tensor_cores=False` keeps every product in fp32 library products.  `with_planes`: returns
    (Q, operand planes of Q or None) - the accumulation keeps the planes of Q in step with its fp32
    form anyway, so a caller that multiplies by Q next need not split it again.  The planes of X carry one
    exponent per matrix, fixed when X is first split: Householder reflections preserve column
    norms, so no entry of the trailing matrix outgrows sqrt(n) times the largest entry of X, which
    the split's headroom (largest entry below 2^9 of fp16's 2^16) covers up to n = 16384.

    The chain of 32-column panel launches is the critical path (a panel kernel occupies one SM
    per matrix for 30-150 us whatever the batch).  With LOOKAHEAD only the update of the NEXT
    outer block's 128 columns stays on it; the rest of each far update runs on a side stream beside
    the next block's panels, and Q is accumulated forwards on a second side stream,
    Q <- Q (I - V T V^T) per finished block (1.5x the flops of the backward accumulation over
    shrinking windows, but off the critical path), so that Q is ready when the last panel is.
    The side-stream products run on a capped number of CTAs (_background_ctas) so that the panel
    kernel always finds free SMs.  The choice of path depends on the order and on whether the batch
    leaves SMs free at all (more than ~100 matrices do not), not otherwise on the batch: a matrix gets
    the same bits whether it is factored alone, in a shard or in the full class."""
    B, n, _ = X.shape
    if X.is_cuda and n > MAX_ORDER:
        global _WARNED_LARGE
        if not _WARNED_LARGE:
            _WARNED_LARGE = True
            warnings.warn(f"householder_q: order {n} exceeds the panel kernel's {MAX_ORDER} rows (a panel must fit one SM's "
                          "shared memory); using torch.linalg.qr for this order - per-matrix library QR, much slower")
        Q = torch.linalg.qr(X).Q
        return (Q, None) if with_planes else Q
    if (not X.is_cuda) or n < 2:
        Q = torch.linalg.qr(X).Q
        return (Q, None) if with_planes else Q
    F._require_lib(X)
    X = X.contiguous()
    lib = F.lib
    from optimizers import _gemm
    tc = USE_TENSOR_CORES and tensor_cores
    npan = (n + PANEL - 1) // PANEL
    V = torch.zeros(B, n, n, dtype=torch.float32, device=X.device)
    T = torch.empty(B, npan, PANEL, PANEL, dtype=torch.float32, device=X.device)
    blocks = []                                           # (J0, wo, T_big, planes of V)
    split = _gemm.split
    side_ctas = _background_ctas(X.device, B) if tc else 0
    lookahead = tc and LOOKAHEAD and n > 2 * OUTER and side_ctas > 0
    forward_q = lookahead and FORWARD_Q
    keep = []                                             # tensors used on side streams stay alive until the join
    with torch.cuda.device(X.device):
        main = torch.cuda.current_stream(X.device)
        stream = F._stream(X)
        rest_stream, q_stream = _side_streams(X.device) if lookahead else (None, None)
        rest_done = None                                  # event: the previous block's remainder update
        Xp = split(X) if tc else None
        Q = Qp = None
        if forward_q:
            Q = torch.eye(n, dtype=torch.float32, device=X.device).expand(B, n, n).contiguous()
            Qp = split(Q, bound=2.0)                      # Q stays orthonormal: entries <= 1
            q_stream.wait_stream(main)
        for J0 in range(0, n, OUTER):
            wo = min(OUTER, n - J0)
            widths = []
            for j0 in range(J0, J0 + wo, PANEL):
                w = min(PANEL, n - j0)
                k = j0 // PANEL
                # each launch first applies the previous panel's reflector to the rest of the outer
                # block (32-column chunks on separate CTAs), then factors its own panel
                prev = PANEL if j0 > J0 else 0
                rc = lib.qt_householder_panel_fused(_ptr(X), n * n, n, B, j0, w, _ptr(V), n * n,
                                                    _ptr(T[:, k]), npan * PANEL * PANEL, prev,
                                                    _ptr(T[:, k - 1]) if prev else None, J0 + wo, stream)
                F._check(rc, "householder panel")
                widths.append(w)
            Vo = V[:, J0:, J0:J0 + wo]
            Pv = split(Vo, bound=2.0) if tc else None     # Householder vectors: entries <= 1; shared by the merge, the far update and the accumulation of Q
            Tb = _merge_t(Vo, T[:, J0 // PANEL:], widths, Pv)
            Pt = split(Tb) if tc else None                # planes of T: shared by the far update (as T^T) and the accumulation of Q
            blocks.append((J0, wo, Tb, Pv, Pt))
            m, t = n - J0, n - J0 - wo
            if not lookahead:
                if t > 0:
                    _reflect(Vo, Tb, X[:, J0:, J0 + wo:], Xp.window(J0, J0 + wo, m, t) if tc else None, True, Pv, Pt)
                continue
            if t == 0 and not forward_q:
                continue
            _, Yp = _gemm.matmul(Pv, Pt, trans_b=True, want_float=False, want_planes=True)     # Y = V T^T
            keep += [Pv, Yp, Tb]
            y_ready = torch.cuda.Event()
            y_ready.record(main)
            if t > 0:
                nxt = min(OUTER, t)                        # the next outer block's columns: needed by its panels
                if rest_done is not None:
                    main.wait_event(rest_done)            # they were last written by the previous block's remainder
                keep.append(_apply_block(Yp, Pv, X[:, J0:, J0 + wo:J0 + wo + nxt], Xp.window(J0, J0 + wo, m, nxt)))
                if t > nxt:
                    rest_stream.wait_event(y_ready)
                    with torch.cuda.stream(rest_stream):
                        keep.append(_apply_block(Yp, Pv, X[:, J0:, J0 + wo + nxt:], Xp.window(J0, J0 + wo + nxt, m, t - nxt), side_ctas))
                        rest_done = torch.cuda.Event()
                        rest_done.record(rest_stream)
            if forward_q:                                 # Q[:, :, J0:] <- Q[:, :, J0:] - (Q[:, :, J0:] V) Y^T
                q_stream.wait_event(y_ready)
                with torch.cuda.stream(q_stream):
                    Qw = Qp.window(0, J0, n, m)
                    _, Wp = _gemm.matmul(Qw, Pv, want_float=False, want_planes=True, max_ctas=side_ctas)
                    _gemm.matmul(Wp, Yp, trans_b=True, alpha=-1.0, beta=1.0, C=Q[:, :, J0:], out=Q[:, :, J0:], out_planes=Qw,
                                 max_ctas=side_ctas)
                    keep.append(Wp)
        if lookahead:
            main.wait_stream(rest_stream)
            if forward_q:
                main.wait_stream(q_stream)
                return (Q, Qp) if with_planes else Q
        Q = torch.eye(n, dtype=torch.float32, device=X.device).expand(B, n, n).contiguous()
        Qp = split(Q, bound=2.0) if tc else None         # Q stays orthonormal: entries <= 1
        for J0, wo, Tb, Pv, Pt in reversed(blocks):
            m = n - J0
            _reflect(V[:, J0:, J0:J0 + wo], Tb, Q[:, J0:, J0:], Qp.window(J0, J0, m, m) if tc else None, False, Pv, Pt)
    return (Q, Qp) if with_planes else Q
