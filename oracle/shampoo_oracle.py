"""CPU oracle of the Shampoo step with low-bit state.  TEST INFRASTRUCTURE ONLY (checker
for tests/, smoke() and the timed CPU baseline of bench.py); the product never imports it.

A per-matrix torch-CPU restatement of the reference's optimizer path, with the C oracle
(oracle/qoracle.c) as the quantizer.  Reference lines followed:

  blocking / reshape       optimizers/shampoo2.py:43-65, :115-121
  eigen-factor state       qtensor/utils.py:126-171 (init, refresh), :192-203 (reconstruct)
  inverse root, mode 0     qtensor/utils.py:205-227 + qtensor/functional.py:749-762
  Schur-Newton             optimizers/matrix_functions.py:22-48, :80-141
  dense-statistic flavour  optimizers/shampoo1.py:148-201
  apply + grafting + tail  optimizers/shampoo2.py:234-272, :441-468 (AdamW), :352-367 (SGD)

Parity is pinned: tests/test_oracle_optimizer.py checks this file against parameters
produced by the reference optimizers themselves (tests/golden/optimizer_cases.npz), in the
reference's 32-bit CPU mode, with 4-bit state forced, and with the reference's diagreal
dequantizer returning None (`diagreal_none=True` reproduces that behaviour).
"""
import itertools
import math

import numpy as np
import torch

from oracle import qoracle


class QState:
    """One blockwise-quantized square matrix (codes + scales [+ fp32 diagonal]) or, when
    plain, the fp32 matrix itself."""

    def __init__(self, mat, bits, blocksize, min_lowbit_size, code, diagreal):
        self.n = mat.shape[0]
        self.lowbit = bits in (4, 8) and mat.numel() >= min_lowbit_size
        self.bits, self.blocksize, self.code, self.diagreal = bits, blocksize, code, diagreal
        self.store(mat)

    def store(self, mat):
        if not self.lowbit:
            self.mat = mat.float().clone()
            return
        res = qoracle.quantize(mat.float().contiguous().numpy(), self.code, self.n, self.blocksize, self.bits,
                               store_diag=self.diagreal)
        self.packed, self.absmax = res[0], res[1]
        self.diag = res[2] if self.diagreal else None

    def load(self):
        if not self.lowbit:
            return self.mat
        out = qoracle.dequantize(self.packed, self.code, self.n, self.absmax, self.blocksize, self.bits,
                                 diag=self.diag)
        return torch.from_numpy(out)


def bjorck(M):
    return 1.5 * M - 0.5 * M @ M.T @ M


def power_iter(G, tol=1e-6, iters=10, v0=None):
    v = (torch.rand(G.shape[0]) * 2 - 1) if v0 is None else v0.clone()
    err, k, sval = 1, 0, 0
    while err > tol and k < iters:
        v = v / torch.norm(v)
        gv = torch.mv(G, v)
        s = torch.dot(v, gv)
        err = torch.abs(s - sval)
        v, sval = gv, s
        k += 1
    return sval


def mat_power(M, p):
    assert p in (1, 2, 4, 8)
    out, done = M, 1
    while done < p:
        out = out @ out
        done *= 2
    return out


def newton_inverse_root(G, p, iters=10, tol=1e-6, ridge=1e-6, v0=None):
    """(G + ridge*lambda_max*I)^(-1/p), coupled Newton iteration (matrix_functions.py:80-141)."""
    n = G.shape[0]
    eye = torch.eye(n)
    if n == 1:
        return eye
    alpha = -1.0 / p
    G = G + ridge * power_iter(G, v0=v0) * eye
    z = (1 + p) / (2 * torch.norm(G))
    root = eye * torch.pow(z, 1.0 / p)
    M = G * z
    err = torch.max(torch.abs(M - eye))
    k = 0
    while err > tol and k < iters:
        T = (1 - alpha) * eye + alpha * M
        cand = root @ T
        M = mat_power(T, p) @ M
        new_err = torch.max(torch.abs(M - eye))
        if new_err > err * 1.2:
            break
        root, err = cand, new_err
        k += 1
    return root


class EigenFactorStat:
    """shampoo2 statistic: quantized basis Vt + lower half of the spectrum.
    cfg["wide"]: every product and the QR run in float64 and only what the reference STORES
    (4-bit codes of fp32 values, fp32 spectrum) is rounded - the exact-arithmetic twin used by
    the tests to measure how far fp32 evaluation order alone moves the result."""

    def __init__(self, n, eps, cfg):
        self.n, self.cfg = n, cfg
        self.wt = torch.float64 if cfg.get("wide") else torch.float32
        self.keep = max(1, n // 2)
        self.keep_idx = torch.arange(self.keep)
        self.S = torch.full((self.keep,), eps, dtype=torch.float32)
        self.max_eig = torch.tensor(eps, dtype=torch.float32)
        self.q = QState(torch.eye(n), cfg["bits"], cfg["blocksize"], cfg["min_lowbit_size"], cfg["code"], False)

    def reconstruct(self):
        Vt = self.q.load().to(self.wt)
        if self.q.lowbit:
            for _ in range(self.cfg["rect_t1"]):
                Vt = bjorck(Vt)
        rows = Vt[self.keep_idx]
        return rows.T @ self.S.to(self.wt).diag() @ rows, Vt

    def refresh(self, L, Vt):
        V, _ = torch.linalg.qr(L @ Vt.T)
        eigs = (V.T @ L @ V).diag()
        vals, idx = torch.sort(eigs)
        self.keep_idx, self.S = idx[: self.keep], vals[: self.keep].float()
        self.max_eig = eigs.max().float()
        self.q.store(V.T.contiguous().float())

    def inverse_root(self, p, eps):
        Vt = self.q.load().to(self.wt)
        rows = Vt[self.keep_idx]
        if self.q.lowbit:
            for _ in range(self.cfg["rect_t2"]):
                rows = bjorck(rows)
        w = 1 / (self.S + eps * self.max_eig).pow(1 / p)
        return (rows.T @ w.to(self.wt).diag() @ rows).float()


def split_sizes(d, block):
    if block > 0 and d > block:
        full, rest = divmod(d, block)
        return [block] * full + ([rest] if rest else [])
    return [d]


class ParamState:
    def __init__(self, shape, cfg):
        self.shape = tuple(shape)
        dims = [x for x in shape if x != 1]
        self.mat_shape = (dims[0], int(np.prod(dims[1:]))) if len(dims) > 1 else None
        self.step = 0
        self.active = False
        self.stats, self.precs, self.blocks = [], [], []
        if self.mat_shape is None:
            return
        cuts = [split_sizes(d, cfg["prec_maxorder"]) for d in self.mat_shape]
        offs = [[0] + list(itertools.accumulate(c)) for c in cuts]
        for i, j in itertools.product(range(len(cuts[0])), range(len(cuts[1]))):
            self.blocks.append((slice(offs[0][i], offs[0][i + 1]), slice(offs[1][j], offs[1][j + 1])))
            for n in (cuts[0][i], cuts[1][j]):
                if cfg["flavour"] == "s2":
                    self.stats.append(EigenFactorStat(n, cfg["matrix_eps"], cfg))
                else:
                    self.stats.append(QState(cfg["matrix_eps"] * torch.eye(n), cfg["bits"], cfg["blocksize"],
                                             cfg["min_lowbit_size"], cfg["code"], True))
                self.precs.append(QState(torch.eye(n), cfg["bits"], cfg["blocksize"], cfg["min_lowbit_size"],
                                         cfg["code"], True))


class OracleShampoo:
    """Steps a list of fp32 CPU tensors in place.  `kind` is 'adamw' or 'sgd'."""

    def __init__(self, params, kind="adamw", flavour="s2", lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.0, momentum=0.9, nesterov=False, start_prec_step=1, stat_compute_steps=100,
                 prec_compute_steps=500, stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200, prec_bits=32,
                 min_lowbit_size=4096, quan_blocksize=64, rect_t1=1, rect_t2=4, inv_root_mode=0,
                 diagreal_none=False, alternate_rounding=False, wide_arithmetic=False):
        self.params = params
        self.kind, self.h = kind, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, momentum=momentum,
                                       nesterov=nesterov, start=start_prec_step, t1=stat_compute_steps,
                                       t2=prec_compute_steps, decay=stat_decay, inv_root_mode=inv_root_mode)
        code = qoracle.linear_map(True, prec_bits, 2) if prec_bits in (4, 8) else None
        self.cfg = dict(flavour=flavour, bits=prec_bits, blocksize=quan_blocksize, min_lowbit_size=min_lowbit_size,
                        code=code, rect_t1=rect_t1, rect_t2=rect_t2, matrix_eps=matrix_eps,
                        prec_maxorder=prec_maxorder, wide=wide_arithmetic)
        # float64 twin (shampoo2 flavour, inverse-root mode 0 only): see EigenFactorStat
        self.wt = torch.float64 if wide_arithmetic else torch.float32
        self.diagreal_none = diagreal_none
        # Sensitivity yardstick for tests: evaluates the statistics update beta*L + (1-beta)*S in
        # another, algebraically identical order (one fp32 rounding differs per element).  How far the
        # parameters move under that change is how finely ANY implementation can be compared
        # with the reference on the same inputs.
        self.alternate_rounding = alternate_rounding
        self.state = [None] * len(params)

    def _load_diagreal(self, q):
        """The reference's low-bit diagreal dequantizer returns None (functional.py:312-368)."""
        if self.diagreal_none and q.lowbit:
            return None
        return q.load()

    def _add_statistics(self, st, grad):
        w1 = self.h["decay"]
        w2 = 1.0 if w1 == 1.0 else 1.0 - w1
        G2 = grad.reshape(st.mat_shape)
        for j, (rs, cs) in enumerate(st.blocks):
            g = G2[rs, cs].to(self.wt)
            for axis in range(2):
                stat = g.T @ g if axis == 1 else g @ g.T
                s = st.stats[2 * j + axis]
                if self.cfg["flavour"] == "s2":
                    L, Vt = s.reconstruct()
                    if self.alternate_rounding:
                        L = L * w1 + w2 * stat
                    else:
                        L.mul_(w1).add_(stat, alpha=w2)       # same operation order as shampoo2.py:199
                    s.refresh(L, Vt)
                else:
                    L = self._load_diagreal(s)
                    if L is None:
                        L = self.cfg["matrix_eps"] * torch.eye(stat.shape[0])
                    s.store(L * w1 + w2 * stat)

    def _compute_preconditioners(self, st):
        eps = self.cfg["matrix_eps"]
        for s, pq in zip(st.stats, st.precs):
            if self.cfg["flavour"] == "s2":
                if self.h["inv_root_mode"] == 0:
                    P = s.inverse_root(4, eps)
                else:
                    P = newton_inverse_root(s.reconstruct()[0].float(), 4, ridge=eps)
            else:
                L = self._load_diagreal(s)
                if L is None:
                    L = eps * torch.eye(pq.n)
                P = newton_inverse_root(L.float(), 4, ridge=eps)
            pq.store(P)
        st.active = True

    def _preconditioned(self, st, grad):
        if not st.precs:
            return grad
        G2 = grad.reshape(st.mat_shape)
        out = torch.empty_like(G2)
        for j, (rs, cs) in enumerate(st.blocks):
            g = G2[rs, cs]
            P0 = self._load_diagreal(st.precs[2 * j])
            P1 = self._load_diagreal(st.precs[2 * j + 1])
            P0 = torch.eye(g.shape[0]) if P0 is None else P0
            P1 = torch.eye(g.shape[1]) if P1 is None else P1
            out[rs, cs] = ((P0.to(self.wt) @ g.to(self.wt)) @ P1.to(self.wt)).to(out.dtype)
        return out.reshape(grad.shape)

    def step(self, grads):
        h = self.h
        for i, (p, grad) in enumerate(zip(self.params, grads)):
            if grad is None:
                continue
            if self.state[i] is None:
                st = self.state[i] = ParamState(p.shape, self.cfg)
                st.m1 = torch.zeros_like(p)
                st.m2 = torch.zeros_like(p)
            st = self.state[i]
            st.step += 1
            if self.kind == "adamw":
                p.mul_(1 - h["lr"] * h["weight_decay"])
            if st.step % h["t1"] == 0 and st.stats:
                self._add_statistics(st, grad)
            if st.step % h["t2"] == 0:
                self._compute_preconditioners(st)
            d = grad
            if st.step >= h["start"] and st.active:
                d = self._preconditioned(st, grad)
                d.mul_(grad.norm() / (d.norm() + 1e-12))
            if self.kind == "adamw":
                b1, b2 = h["betas"]
                st.m1.mul_(b1).add_(d, alpha=1 - b1)
                st.m2.mul_(b2).addcmul_(d, d, value=1 - b2)
                denom = (st.m2.sqrt() / math.sqrt(1 - b2 ** st.step)).add_(h["eps"])
                p.addcdiv_(st.m1, denom, value=-(h["lr"] / (1 - b1 ** st.step)))
            else:
                if h["weight_decay"] != 0.0:
                    d.add_(p, alpha=h["weight_decay"])
                st.m1.mul_(h["momentum"]).add_(d)
                upd = d.add(st.m1, alpha=h["momentum"]) if h["nesterov"] else st.m1
                p.add_(upd, alpha=-h["lr"])
