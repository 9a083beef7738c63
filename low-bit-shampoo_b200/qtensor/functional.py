"""Blockwise quantize / dequantize entry points backed by libqtensor_b200.so.

Same names, argument order and return values as the reference's qtensor/functional.py
(:68 get_ptr, :87 create_dynamic_map, :106 create_linear_map, :116 quantize_blockwise,
:181 dequantize_blockwise, :239 quantize_blockwise_diagreal,
:312 dequantize_blockwise_diagreal, :749 compute_power).  Differences, all deliberate:

* only CUDA tensors are accepted.  The reference falls back to Python loops on CPU and
  MPS; this package has a single sm_100a path and raises RuntimeError otherwise;
* the kernels run on torch's current stream of the tensor's device (the reference always
  uses the legacy default stream, cudaC_python/csrc/ops.cu:59);
* the byte format is the one of the reference's CPU quantizer (:526-746): element 2j
  in the high nibble of byte j, all-zero blocks store index 0, IEEE division by absmax,
  ties to the lower code;
* dequantize_blockwise_diagreal returns the matrix.  The reference's function ends
  without a return statement (:312-368) although every branch fills `out`.
"""
import ctypes as ct
import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from qtensor.cextension import get_lib

try:
    lib = get_lib()
    _lib_error = None
except Exception as exc:                      # reported when a CUDA entry point is used
    lib = None
    _lib_error = exc

_BLOCKSIZES = (2048, 1024, 512, 256, 128, 64)
_DTYPE_TAG = {torch.float32: 0, torch.bfloat16: 1}


def get_ptr(A: Optional[Tensor]) -> Optional[ct.c_void_p]:
    """ctypes pointer to the first element of a tensor (None passes through)."""
    return None if A is None else ct.c_void_p(A.data.data_ptr())


def create_dynamic_map(signed=True, total_bits=8, power=1):
    """Codebook with exponentially spaced decades (reference functional.py:87-103)."""
    ebits = total_bits - 1
    entries = []
    for i in range(ebits):
        count = int(2 ** i + 1 if signed else 2 ** (i + 1) + 1)
        edges = torch.linspace(0.1, 1, count)
        centres = (edges[:-1] + edges[1:]) / 2.0
        decade = 10 ** (-(ebits - 1) + i)
        entries += (decade * centres).tolist()
        if signed:
            entries += (-decade * centres).tolist()
    entries += [0, 1.0]
    entries.sort()
    t = torch.Tensor(entries)
    return t.sign() * t.abs().pow(power)


def create_linear_map(signed=True, total_bits=8, power=2):
    """Evenly spaced points on [-1, 1] raised to `power` with their sign kept; the entry
    just below the middle is an exact zero (reference functional.py:106-113)."""
    n = 2 ** total_bits
    if signed:
        pts = torch.linspace(-1, 1, n)
        pts[n // 2 - 1] = 0
    else:
        pts = torch.linspace(0, 1, n)
    return pts.sign() * pts.abs().pow(power)


def _require_lib(t: Tensor):
    if not t.is_cuda:
        raise RuntimeError(
            f"qtensor (B200 build) only runs on CUDA tensors; got a tensor on {t.device}. "
            "There is no CPU or MPS path in this package.")
    if lib is None:
        raise RuntimeError(
            "CUDA quantization library is unavailable; rebuild the extension "
            f"(csrc/build.py). Loader error: {_lib_error}")


def _num_blocks(order: int, blocksize: int) -> int:
    return order * ((order + blocksize - 1) // blocksize)


def _packed_numel(order: int, bits: int) -> int:
    per_byte = 8 // bits
    return (order * order + per_byte - 1) // per_byte


# QT_CHECK_EACH_CALL=1: synchronise after every library call and read the device status word, so
# that a kernel-side error (a bounded wait that ran out, a value outside an operand plane's range)
# is reported by the call that caused it instead of at the next periodic check.  Debugging aid:
# it serialises the step and cannot be used while a CUDA graph is being captured.
CHECK_EACH_CALL = os.environ.get("QT_CHECK_EACH_CALL", "0") == "1"


def _check(status: int, what: str):
    if status != 0:
        raise RuntimeError(f"{what} failed: {lib.qt_error_string(status).decode()} (status {status})")
    if CHECK_EACH_CALL and not torch.cuda.is_current_stream_capturing():
        torch.cuda.synchronize()
        rc = lib.qt_device_error(1)
        if rc != 0:
            raise RuntimeError(f"{what}: device status {rc} ({lib.qt_error_string(rc).decode()})")


def _stream(t: Tensor) -> ct.c_void_p:
    return ct.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _quantize(A, code, order, absmax, diag, out, blocksize, bits, diagreal):
    _require_lib(A)
    if absmax is None:
        absmax = torch.empty((_num_blocks(order, blocksize),), device=A.device, dtype=torch.float32)
    if diagreal and diag is None:
        diag = torch.empty((order,), device=A.device, dtype=torch.float32)
    if out is None:
        out = torch.empty(_packed_numel(order, bits), device=A.device, dtype=torch.uint8)
    assert blocksize in _BLOCKSIZES
    assert code.shape == torch.Size([2 ** bits])
    if A.dtype not in _DTYPE_TAG:
        raise ValueError(f"data type of A is not supported: {A.dtype}")
    with torch.cuda.device(A.device):
        status = lib.qt_quantize_blockwise(
            get_ptr(A), _DTYPE_TAG[A.dtype], 0, get_ptr(code), order, 1,
            get_ptr(absmax), 0, get_ptr(diag) if diagreal else None, 0,
            get_ptr(out), 0, blocksize, bits, _stream(A))
    _check(status, "quantize_blockwise")
    return out, absmax, diag


def _dequantize(A, code, order, absmax, diag, outdtype, out, blocksize, bits, diagreal):
    _require_lib(A)
    if out is None:
        out = torch.empty((order, order), device=A.device, dtype=outdtype)
    assert blocksize in _BLOCKSIZES
    assert code.shape == torch.Size([2 ** bits])
    if out.dtype not in _DTYPE_TAG:
        raise ValueError(f"data type of out is not supported: {out.dtype}")
    with torch.cuda.device(A.device):
        status = lib.qt_dequantize_blockwise(
            get_ptr(A), 0, get_ptr(code), order, 1, get_ptr(absmax), 0,
            get_ptr(diag) if diagreal else None, 0,
            get_ptr(out), _DTYPE_TAG[out.dtype], 0, blocksize, bits, _stream(A))
    _check(status, "dequantize_blockwise")
    return out


def quantize_blockwise(
    A: Tensor,
    code: Tensor,
    order: int,
    absmax: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 256,
    bits: int = 8,
) -> Tuple[Tensor, Tensor]:
    """Quantize the contiguous row-major (order, order) matrix A; returns (codes, absmax)."""
    out, absmax, _ = _quantize(A, code, order, absmax, None, out, blocksize, bits, False)
    return out, absmax


def dequantize_blockwise(
    A: Tensor,
    code: Tensor,
    order: int,
    absmax: Tensor,
    outdtype=torch.float32,
    out: Optional[Tensor] = None,
    blocksize: int = 256,
    bits: int = 8,
) -> Tensor:
    """Inverse of quantize_blockwise; returns the (order, order) matrix of dtype outdtype."""
    return _dequantize(A, code, order, absmax, None, outdtype, out, blocksize, bits, False)


def quantize_blockwise_diagreal(
    A: Tensor,
    code: Tensor,
    order: int,
    absmax: Optional[Tensor] = None,
    diag: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 256,
    bits: int = 8,
) -> Tuple[Tensor, Tensor, Tensor]:
    """As quantize_blockwise, with the diagonal kept in fp32 and left out of scales and codes."""
    return _quantize(A, code, order, absmax, diag, out, blocksize, bits, True)


def dequantize_blockwise_diagreal(
    A: Tensor,
    code: Tensor,
    order: int,
    absmax: Tensor,
    diag: Tensor,
    outdtype=torch.float32,
    out: Optional[Tensor] = None,
    blocksize: int = 256,
    bits: int = 8,
) -> Tensor:
    """Inverse of quantize_blockwise_diagreal (diagonal restored from `diag`)."""
    return _dequantize(A, code, order, absmax, diag, outdtype, out, blocksize, bits, True)


@torch.no_grad()
def ridged_inverse_root(S, rho, p):
    """(S + rho)^(-1/p) as in the reference (functional.py:760-762) wherever S + rho > 0.  The S are
    Rayleigh quotients of a positive semi-definite statistic computed in fp32: rounding can
    leave one at or below -rho (seen after ten identical gradients on a 768 x 384 block, where the
    kept half of the spectrum is pure ridge), which the reference turns into inf or NaN that then
    spreads over the parameter.  Such an entry is treated as the zero it stands for:
    rho^(-1/p).  `rho` broadcasts against the last dimension of S."""
    t = S + rho
    return 1 / torch.where(t > 0, t, rho.expand_as(t) if torch.is_tensor(rho) else torch.full_like(t, rho)).pow(1 / p)


@torch.no_grad()
def compute_power(Vt, S, p, iter_count=4, ridge_epsilon=1e-6, indices=None, max_eigen=None):
    """Inverse p-th root from an eigen-factor form: rows `indices` of Vt are rectified by
    `iter_count` Bjorck steps, then  rows^T diag((S + ridge * lambda_max)^(-1/p)) rows
    (reference functional.py:749-762; lambda_max defaults to max(S))."""
    rows = Vt[indices] if indices is not None else Vt
    top = max_eigen if max_eigen is not None else S.max()
    weights = ridged_inverse_root(S, ridge_epsilon * top, p)
    if rows.is_cuda and rows.dtype == torch.float32 and lib is not None:
        # the same products on the tensor cores (batch of one; fp32 results re-split between
        # products, so any input is accepted - the optimizers' batched engine chains planes instead)
        from optimizers import _engine as E
        R = E.Mat(rows.contiguous().unsqueeze(0))
        for _ in range(iter_count):
            W = E.mm(R, R, trans_b=True)
            R = E.mm(W, R, alpha=-0.5, beta=1.5, C=R.f32)
        scaled = E.Mat((weights.to(rows.device).unsqueeze(1) * R.f32[0]).unsqueeze(0))
        return E.mm(R, scaled, trans_a=True).f32[0]
    for _ in range(iter_count):
        rows = torch.addmm(rows, rows @ rows.T, rows, beta=1.5, alpha=-0.5)
    return rows.T @ (weights.unsqueeze(1) * rows)
