"""Matrix helpers of the Schur-Newton inverse-root path.

Same names and return values as the reference's optimizers/matrix_functions.py
(PowerIter :22-48, MatPower :52-76, ComputePower :80-141).  Each function also accepts a
batch (m, n, n): every matrix follows its own stopping rule, so a whole order class runs
together with no per-matrix host synchronisation (the reference synchronises twice per
Newton iteration per matrix, :131,:136).

CUDA fp32 input runs inside the native library: one fused power-iteration kernel, then the
Newton chain root T, T^2, T^4, T^4 M as three-plane tcgen05 products whose epilogues write
the next product's operands, reduce max |M - I| and obey per-matrix accept / stop flags in
device memory (qt_inverse_root_newton).  CPU tensors (the 32-bit mode the reference itself runs
in on CPU) take the batched torch statement of the same algorithm below.
"""
import ctypes as ct

import torch

import qtensor.functional as F

# Where the start vector of the power iteration comes from when the caller gives none.  The
# reference draws torch.rand(n, device=mat.device) * 2 - 1 once per matrix (:36), i.e. from the
# generator of the matrix's device: "device" does exactly that, one draw per matrix in batch
# order.  "host" draws from the CPU generator instead (what the reference does when it runs on CPU
# tensors); it exists so that a CUDA run can be compared with CPU-generated reference results and
# is not usable under CUDA-graph capture.
START_VECTORS = "device"
_WORKSPACE_CAP = 6 << 30           # bytes of Newton workspace per launch group; larger batches are cut


def _ptr(t):
    return None if t is None else ct.c_void_p(t.data_ptr())


def draw_start_vectors(m, n, device):
    """m start vectors of length n, uniform in (-1, 1), drawn one matrix at a time (the reference's order)."""
    if START_VECTORS == "host" or torch.device(device).type != "cuda":
        return torch.stack([torch.rand(n) * 2 - 1 for _ in range(m)]).to(device)
    return torch.stack([torch.rand(n, device=device) * 2 - 1 for _ in range(m)])


def _native(G):
    return (G.is_cuda and G.dtype == torch.float32 and F.lib is not None and G.shape[-1] >= 2 and G.shape[-1] <= 25000)


@torch.no_grad()
def PowerIter(mat_g, error_tolerance=1e-6, num_iters=10, v0=None):
    """Largest eigenvalue by power iteration from a start vector uniform in (-1, 1).

    Returns (eigenvalue, unit vector, iterations).  `v0` fixes the start vector (the
    reference always draws torch.rand, :36).  For a batch, `iterations` is a tensor.
    """
    batched = mat_g.dim() == 3
    G = mat_g if batched else mat_g.unsqueeze(0)
    m, n = G.shape[0], G.shape[-1]
    if v0 is None:
        v = draw_start_vectors(m, n, G.device)
    else:
        v = v0.reshape(m, n).to(G.device, torch.float32).clone()
    if _native(G):
        Gc = G.contiguous()
        v = v.contiguous()
        sval = torch.empty(m, device=G.device)
        iters = torch.empty(m, dtype=torch.int32, device=G.device)
        vec = torch.empty(m, n, device=G.device)
        with torch.cuda.device(G.device):
            rc = F.lib.qt_power_iter(_ptr(Gc), n * n, n, m, _ptr(v), float(error_tolerance), int(num_iters),
                                     _ptr(sval), _ptr(iters), _ptr(vec), F._stream(Gc))
        F._check(rc, "power iteration")
        vec = vec / torch.linalg.vector_norm(vec, dim=1, keepdim=True)
        if batched:
            return sval, vec, iters.to(torch.int64)
        return sval[0], vec[0], int(iters[0])
    sval = torch.zeros(m, device=G.device)
    active = torch.ones(m, dtype=torch.bool, device=G.device)
    iters = torch.zeros(m, dtype=torch.int64, device=G.device)
    for _ in range(num_iters):
        vn = v / torch.linalg.vector_norm(v, dim=1, keepdim=True)
        gv = torch.bmm(G, vn.unsqueeze(2)).squeeze(2)
        s = (vn * gv).sum(dim=1)
        err = (s - sval).abs()
        v = torch.where(active.unsqueeze(1), gv, v)
        sval = torch.where(active, s, sval)
        iters += active
        active = active & (err > error_tolerance)
    vec = v / torch.linalg.vector_norm(v, dim=1, keepdim=True)
    if batched:
        return sval, vec, iters
    return sval[0], vec[0], int(iters[0])


def _mm(a, b):
    """a @ b for batches; CUDA fp32 operands run on the three-plane tcgen05 product."""
    if a.dim() == 3 and _native(a) and a.shape == b.shape:
        from optimizers import _gemm
        D, _ = _gemm.matmul(_gemm.split3(a.contiguous()), _gemm.split3(b.contiguous()))
        return D
    return torch.matmul(a, b)


@torch.no_grad()
def MatPower(mat_m, p):
    """mat_m ** p for a positive integer p (repeated squaring)."""
    single = mat_m.dim() == 2
    M = mat_m.unsqueeze(0) if single else mat_m
    if p in (1, 2, 4, 8, 16, 32):
        out, done = M, 1
        while done < p:
            out = _mm(out, out)
            done *= 2
    else:
        out = None
        while p > 0:
            if p % 2 == 1:
                out = _mm(M, out) if out is not None else M
            p //= 2
            M = _mm(M, M)
    return out[0] if single else out


def _compute_power_native(G, p, iter_count, error_tolerance, ridge_epsilon, v0):
    """Batched inverse root inside the library.  G: (m, n, n) CUDA fp32 contiguous, modified in place."""
    m, n = G.shape[0], G.shape[-1]
    lib = F.lib
    out = torch.empty_like(G)
    per = int(lib.qt_inverse_root_newton_workspace_bytes(n, 1))
    chunk = max(1, min(m, _WORKSPACE_CAP // max(per, 1)))
    with torch.cuda.device(G.device):
        for a in range(0, m, chunk):
            b = min(m, a + chunk)
            need = int(lib.qt_inverse_root_newton_workspace_bytes(n, b - a))
            ws = torch.empty(need, dtype=torch.uint8, device=G.device)
            rc = lib.qt_inverse_root_newton(_ptr(G[a:b]), n * n, n, b - a, int(p), int(iter_count), float(error_tolerance),
                                            float(ridge_epsilon), _ptr(v0[a:b]), _ptr(ws), need, _ptr(out[a:b]), n * n,
                                            None, None, F._stream(G))
            F._check(rc, "inverse root (Newton)")
    return out


@torch.no_grad()
def ComputePower(mat_g, p, iter_count=10, error_tolerance=1e-6, ridge_epsilon=1e-6, v0=None):
    """(mat_g + r I)^(-1/p), r = ridge_epsilon * lambda_max(mat_g), by the coupled Newton
    iteration of Guo & Higham (2006), eq. 3.2.  mat_g is modified in place (ridge added),
    as in the reference (:112).  A 1-D input is treated as a diagonal."""
    if mat_g.dim() == 1:
        return torch.pow(mat_g + ridge_epsilon, -1 / p)
    batched = mat_g.dim() == 3
    G = mat_g if batched else mat_g.unsqueeze(0)
    m, n = G.shape[0], G.shape[-1]
    eye = torch.eye(n, device=G.device)
    if n == 1:
        return eye.expand(m, 1, 1).clone() if batched else eye
    if _native(G) and G.is_contiguous() and p >= 2 and (p & (p - 1)) == 0 and p <= 64:
        if v0 is None:
            v0 = draw_start_vectors(m, n, G.device)
        v0 = v0.reshape(m, n).to(G.device, torch.float32).contiguous()
        root = _compute_power_native(G, p, iter_count, error_tolerance, ridge_epsilon, v0)
        return root if batched else root[0]
    alpha = -1.0 / p
    max_ev, _, _ = PowerIter(G, v0=v0)
    G.diagonal(dim1=1, dim2=2).add_((ridge_epsilon * max_ev).unsqueeze(1))
    z = (1 + p) / (2 * torch.linalg.matrix_norm(G))            # Frobenius, per matrix
    root = eye * torch.pow(z, 1.0 / p).view(m, 1, 1)
    M = G * z.view(m, 1, 1)
    err = (M - eye).abs().amax(dim=(1, 2))
    active = err > error_tolerance
    for _ in range(iter_count):
        if not bool(active.any()):
            break
        T = (1 - alpha) * eye + alpha * M
        new_root = torch.matmul(root, T)
        new_M = torch.matmul(MatPower(T, p), M)
        new_err = (new_M - eye).abs().amax(dim=(1, 2))
        accept = active & ~(new_err > err * 1.2)
        sel = accept.view(m, 1, 1)
        root = torch.where(sel, new_root, root)
        M = torch.where(sel, new_M, M)
        err = torch.where(accept, new_err, err)
        active = accept & (err > error_tolerance)
    return root if batched else root[0]
