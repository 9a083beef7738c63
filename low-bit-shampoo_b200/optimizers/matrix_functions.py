"""Matrix helpers of the Schur-Newton inverse-root path.

Same names and return values as the reference's optimizers/matrix_functions.py
(PowerIter :22-48, MatPower :52-76, ComputePower :80-141).  Each function also accepts a
batch (m, n, n): every matrix follows its own stopping rule through masks, so a whole
order class runs as batched products with no per-matrix host synchronisation (the
reference synchronises twice per Newton iteration per matrix, :131,:136).
"""
import torch


def _bmm(a, b):
    return torch.matmul(a, b)


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
        v = torch.rand(m, n, device=G.device) * 2 - 1
    else:
        v = v0.reshape(m, n).to(G.device, torch.float32).clone()
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


@torch.no_grad()
def MatPower(mat_m, p):
    """mat_m ** p for a positive integer p (repeated squaring)."""
    if p in (1, 2, 4, 8, 16, 32):
        out, done = mat_m, 1
        while done < p:
            out = _bmm(out, out)
            done *= 2
        return out
    acc = None
    while p > 0:
        if p % 2 == 1:
            acc = _bmm(mat_m, acc) if acc is not None else mat_m
        p //= 2
        mat_m = _bmm(mat_m, mat_m)
    return acc


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
        new_root = _bmm(root, T)
        new_M = _bmm(MatPower(T, p), M)
        new_err = (new_M - eye).abs().amax(dim=(1, 2))
        accept = active & ~(new_err > err * 1.2)
        sel = accept.view(m, 1, 1)
        root = torch.where(sel, new_root, root)
        M = torch.where(sel, new_M, M)
        err = torch.where(accept, new_err, err)
        active = accept & (err > error_tolerance)
    return root if batched else root[0]
