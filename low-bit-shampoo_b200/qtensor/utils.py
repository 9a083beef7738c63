"""Holders of quantized preconditioner state (one square matrix each).

Public surface and attribute names follow the reference's qtensor/utils.py:
QTensor (:7-61), QTensorDiagReal (:64-121) and QTensorSVDFast (:124-236) - the
attributes `var`, `absmax`, `diag`, `Svalue`, `keep_indices`, `max_eigenvalue`,
`var_order`, `var_dtype`, `blocksize`, `bits`, `code`, `name2qmap` keep their meaning,
so optimizer state dicts pickle the same objects.

All three accept an optional `storage` dict of preallocated tensors (views into a
larger arena).  The optimizers use it to lay every matrix of one order out contiguously
so that a whole order class is (de)quantized by one batched kernel launch.
"""
import torch

import qtensor.functional as F


def _is_plain(bits, var, min_lowbit_size):
    return bits in (32, 16) or var.numel() < min_lowbit_size


def _plain_tensor(value, bits, storage):
    """Plain (16/32-bit) state: a fresh tensor, or the caller's arena view filled in place."""
    value = value.bfloat16() if bits == 16 else value.float()
    if storage and "var" in storage:
        storage["var"].copy_(value)
        return storage["var"], True
    return value, False


class _LowBitBase:
    """Shared bookkeeping: codebook lookup and buffer adoption."""

    def _setup_lowbit(self, var, name2qmap, code, blocksize):
        name2qmap[code] = name2qmap[code].to(var.device)
        self.name2qmap = name2qmap
        self.code = code
        self.blocksize = blocksize
        self.var_order = var.shape[0]

    def _codebook(self):
        return self.name2qmap[self.code]

    def _drop_buffers_if_order_changed(self, var, names):
        if var.shape[0] != self.var_order:
            self.var_order = var.shape[0]
            self.var_dtype = var.dtype
            for n in names:
                setattr(self, n, None)


class QTensor(_LowBitBase):
    """Plain blockwise-quantized matrix (no side channel)."""

    def __init__(self, var, bits=32, name2qmap={}, code='', blocksize=2048, min_lowbit_size=4096, storage=None):
        self.bits = bits
        self._pinned = False
        if _is_plain(bits, var, min_lowbit_size):
            self.bits = 16 if bits == 16 else 32
            self.var, self._pinned = _plain_tensor(var, self.bits, storage)
        elif bits in (8, 4):
            self._setup_lowbit(var, name2qmap, code, blocksize)
            self.var_dtype = var.dtype
            st = storage or {}
            self.var, self.absmax = F.quantize_blockwise(
                var.contiguous(), code=self._codebook(), order=self.var_order, absmax=st.get("absmax"),
                out=st.get("var"), blocksize=blocksize, bits=bits)
        else:
            raise ValueError(f'num of bits is not supported: {self.bits}')

    def quantize(self, var):
        if self.bits >= 16:
            if self._pinned and var.shape == self.var.shape:
                self.var.copy_(var)
            else:
                self.var = var.to(self.var.dtype)
            return
        self._drop_buffers_if_order_changed(var, ("var", "absmax"))
        self.var, self.absmax = F.quantize_blockwise(
            var.contiguous(), code=self._codebook(), order=self.var_order, absmax=self.absmax,
            out=self.var, blocksize=self.blocksize, bits=self.bits)

    def dequantize(self):
        if self.bits >= 16:
            return self.var
        return F.dequantize_blockwise(self.var, code=self._codebook(), order=self.var_order, absmax=self.absmax,
                                      outdtype=self.var_dtype, blocksize=self.blocksize, bits=self.bits)

    def set_device(self, device):
        if self.bits < 16:
            self.name2qmap[self.code] = self.name2qmap[self.code].to(device)
            self.absmax = self.absmax.to(device)
        self.var = self.var.to(device)


class QTensorDiagReal(_LowBitBase):
    """Blockwise-quantized matrix whose diagonal is kept in fp32 (`diag`) and is excluded
    from the block scales and codes."""

    def __init__(self, var, bits=32, name2qmap={}, code='', blocksize=2048, min_lowbit_size=4096, storage=None):
        self.bits = bits
        self._pinned = False
        if _is_plain(bits, var, min_lowbit_size):
            self.bits = 16 if bits == 16 else 32
            self.var, self._pinned = _plain_tensor(var, self.bits, storage)
        elif bits in (8, 4):
            self._setup_lowbit(var, name2qmap, code, blocksize)
            self.var_dtype = var.dtype
            st = storage or {}
            self.var, self.absmax, self.diag = F.quantize_blockwise_diagreal(
                var.contiguous(), code=self._codebook(), order=self.var_order, absmax=st.get("absmax"),
                diag=st.get("diag"), out=st.get("var"), blocksize=blocksize, bits=bits)
        else:
            raise ValueError(f'num of bits is not supported: {self.bits}')

    def quantize(self, var):
        if self.bits >= 16:
            if self._pinned and var.shape == self.var.shape:
                self.var.copy_(var)
            else:
                self.var = var.to(self.var.dtype)
            return
        self._drop_buffers_if_order_changed(var, ("var", "absmax", "diag"))
        self.var, self.absmax, self.diag = F.quantize_blockwise_diagreal(
            var.contiguous(), code=self._codebook(), order=self.var_order, absmax=self.absmax, diag=self.diag,
            out=self.var, blocksize=self.blocksize, bits=self.bits)

    def dequantize(self):
        if self.bits >= 16:
            return self.var
        return F.dequantize_blockwise_diagreal(
            self.var, code=self._codebook(), order=self.var_order, absmax=self.absmax, diag=self.diag,
            outdtype=self.var_dtype, blocksize=self.blocksize, bits=self.bits)

    def set_device(self, device):
        if self.bits < 16:
            self.name2qmap[self.code] = self.name2qmap[self.code].to(device)
            self.absmax = self.absmax.to(device)
            self.diag = self.diag.to(device)
        self.var = self.var.to(device)


def bjorck_step(M):
    """One Bjorck orthonormalisation step on the rows of M: 1.5 M - 0.5 (M M^T) M."""
    if M.is_cuda and M.dtype == torch.float32 and F.lib is not None:
        from optimizers import _engine as E
        R = E.Mat(M.contiguous().unsqueeze(0))
        return E.mm(E.mm(R, R, trans_b=True), R, alpha=-0.5, beta=1.5, C=R.f32).f32[0]
    return torch.addmm(M, M @ M.T, M, beta=1.5, alpha=-0.5)


class QTensorSVDFast(_LowBitBase):
    """Eigen-factor form of a symmetric PSD statistic L: the rows of `var` (quantized) are
    approximate eigenvectors, `Svalue` / `keep_indices` hold the lower half of the
    spectrum (values and row numbers, ascending) and `max_eigenvalue` the largest one.
    quantize() refreshes the basis with one subspace-iteration step (QR of L V)."""

    def __init__(self, var, bits=32, name2qmap={}, code='', blocksize=2048, min_lowbit_size=4096,
                 rect_t1=1, rect_t2=4, log_prefix=None, storage=None):
        self.bits = bits
        self.rect_t1 = rect_t1
        self.rect_t2 = rect_t2
        # The reference writes logs/eigenvalues_<prefix>.csv on the first quantize()
        # (utils.py:173-189).  That side effect is kept but only when a prefix is given;
        # the optimizers of this package pass None.
        self.log_prefix = log_prefix
        self._log_written = False

        n = var.shape[0]
        keep = max(1, n // 2)
        st = storage or {}
        scale = var[0][0]
        eigs = scale * torch.ones(n, device=var.device, dtype=torch.float32)
        self.keep_indices = torch.arange(keep, device=var.device, dtype=torch.int64)
        self.Svalue = eigs[:keep].clone()
        self.max_eigenvalue = eigs.max().clone()
        if "Svalue" in st:
            st["Svalue"].copy_(self.Svalue); self.Svalue = st["Svalue"]
            st["keep_indices"].copy_(self.keep_indices); self.keep_indices = st["keep_indices"]
            st["max_eigenvalue"].copy_(self.max_eigenvalue); self.max_eigenvalue = st["max_eigenvalue"]

        basis = torch.eye(n, device=var.device)
        self._pinned = False
        if _is_plain(bits, var, min_lowbit_size):
            self.bits = 32
            self.var, self._pinned = _plain_tensor(basis, 32, storage)
        elif bits in (8, 4):
            self._setup_lowbit(var, name2qmap, code, blocksize)
            self.var_dtype = basis.dtype
            self.var, self.absmax = F.quantize_blockwise(
                basis, code=self._codebook(), order=self.var_order, absmax=st.get("absmax"), out=st.get("var"),
                blocksize=blocksize, bits=bits)
        else:
            raise ValueError(f'num of bits is not supported: {self.bits}')

    def _assign(self, name, value):
        cur = getattr(self, name)
        if cur is not None and cur.shape == value.shape and cur.dtype == value.dtype and cur.device == value.device:
            cur.copy_(value)
        else:
            setattr(self, name, value)

    def quantize(self, var, Vt=None):
        L = var.float()
        if L.is_cuda and F.lib is not None and L.shape[0] >= 2:
            # batch of one through the optimizers' engine: L V^T and L V on the tensor cores, the QR
            # on the library's Householder kernels (no cuSOLVER / cuBLAS call)
            from optimizers import _engine as E
            Vb, eb = E.op_subspace_step(E.Mat(L.contiguous().unsqueeze(0)), E.Mat(Vt.float().contiguous().unsqueeze(0)))
            V, eigs = Vb[0], eb[0]
        else:
            V, _ = torch.linalg.qr(L @ Vt.T.float())
            eigs = ((L @ V) * V).sum(dim=0)                   # diag(V^T L V)
        keep = max(1, eigs.numel() // 2)
        order_vals, order_idx = torch.sort(eigs)
        self._assign("keep_indices", order_idx[:keep].to(torch.int64))
        self._assign("Svalue", order_vals[:keep].to(var.dtype))
        self._assign("max_eigenvalue", eigs.max().to(var.dtype))
        if self.bits < 16:
            F.quantize_blockwise(V.T.contiguous(), code=self._codebook(), order=self.var_order, absmax=self.absmax,
                                 out=self.var, blocksize=self.blocksize, bits=self.bits)
        elif self._pinned:
            self.var.copy_(V.T)
        else:
            self.var = V.T.contiguous()
        if self.log_prefix and not self._log_written:
            self._write_spectrum_log(order_vals, keep)

    def _write_spectrum_log(self, ascending_vals, keep):
        import re
        from pathlib import Path
        Path("logs").mkdir(parents=True, exist_ok=True)
        name = re.sub(r"[^A-Za-z0-9_.-]", "_", self.log_prefix)
        with open(Path("logs") / f"eigenvalues_{name}.csv", "w", encoding="utf-8") as f:
            f.write("rank,value\n")
            for i, v in enumerate(ascending_vals.detach().cpu().tolist(), start=1):
                f.write(f"{i},{float(v)}\n")
        self._log_written = True

    def _basis(self, iters):
        if self.bits >= 16:
            return self.var
        Vt = F.dequantize_blockwise(self.var, code=self._codebook(), order=self.var_order, absmax=self.absmax,
                                    outdtype=self.var_dtype, blocksize=self.blocksize, bits=self.bits)
        for _ in range(iters):
            Vt = bjorck_step(Vt)
        return Vt

    def dequantize(self):
        """Returns (L restricted to the kept half of the spectrum, rectified basis Vt)."""
        Vt = self._basis(self.rect_t1)
        rows = Vt[self.keep_indices.to(Vt.device)]
        S = self.Svalue.to(device=Vt.device, dtype=Vt.dtype)
        if rows.is_cuda and rows.dtype == torch.float32 and F.lib is not None:
            from optimizers import _engine as E
            R = E.Mat(rows.contiguous().unsqueeze(0))
            return E.mm(R, E.Mat((S.unsqueeze(1) * rows).unsqueeze(0)), trans_a=True).f32[0], Vt
        return rows.T @ (S.unsqueeze(1) * rows), Vt

    def computepower(self, exp, ridge_epsilon=1e-6):
        """(L + ridge * lambda_max I)^(-1/exp) on the kept half of the spectrum."""
        if self.bits < 16:
            Vt, iters = self._basis(0), self.rect_t2
        else:
            Vt, iters = self.var, 0
        return F.compute_power(Vt, self.Svalue, exp, iter_count=iters, ridge_epsilon=ridge_epsilon,
                               indices=self.keep_indices, max_eigen=self.max_eigenvalue)

    def set_device(self, device):
        if self.bits < 16:
            self.name2qmap[self.code] = self.name2qmap[self.code].to(device)
            self.absmax = self.absmax.to(device)
        self.Svalue = self.Svalue.to(device)
        self.keep_indices = self.keep_indices.to(device)
        self.max_eigenvalue = self.max_eigenvalue.to(device)
        self.var = self.var.to(device)
