"""ctypes/numpy front end of the C oracle in qoracle.c (test infrastructure only).

Mirrors the argument meaning of the reference's CPU quantizer entry points
(qtensor/functional.py:116-178, 181-236, 239-309, 312-368) on numpy arrays:
fp32 matrices are float32 arrays, bf16 matrices are uint16 arrays of bit patterns.
"""
import ctypes as ct
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    """Compile qoracle.c into libqoracle.so next to it (gcc, a second or two)."""
    so = os.path.join(_HERE, "libqoracle.so")
    src = os.path.join(_HERE, "qoracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libqoracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ct.CDLL(build())
        _LIB.qoracle_quantize.restype = ct.c_int
        _LIB.qoracle_dequantize.restype = ct.c_int
    return _LIB


def bf16_bits_to_f32(a):
    """uint16 bf16 bit patterns -> float32 (exact)."""
    return (a.astype(np.uint32) << 16).view(np.float32)


def _ptr(a):
    return ct.c_void_p(a.ctypes.data) if a is not None else ct.c_void_p(0)


def num_blocks(order, blocksize):
    return (order + blocksize - 1) // blocksize


def quantize(A, code, order, blocksize=64, bits=4, store_diag=False):
    """Returns (packed uint8, absmax float32[, diag float32])."""
    if A.dtype == np.uint16:
        A = bf16_bits_to_f32(A)
    A = np.ascontiguousarray(A, dtype=np.float32).reshape(-1)
    assert A.size == order * order
    code = np.ascontiguousarray(code, dtype=np.float32)
    assert code.size == 2 ** bits
    total = order * order
    out = np.zeros(total if bits == 8 else (total + 1) // 2, dtype=np.uint8)
    absmax = np.zeros(order * num_blocks(order, blocksize), dtype=np.float32)
    diag = np.zeros(order, dtype=np.float32) if store_diag else None
    rc = lib().qoracle_quantize(_ptr(A), _ptr(code), ct.c_int(order), ct.c_int(blocksize),
                                ct.c_int(bits), _ptr(absmax), _ptr(diag), _ptr(out))
    if rc != 0:
        raise ValueError("qoracle_quantize rejected its arguments")
    return (out, absmax, diag) if store_diag else (out, absmax)


def dequantize(packed, code, order, absmax, blocksize=64, bits=4, diag=None, out_bf16=False):
    """Returns float32 (order, order), or uint16 bf16 bit patterns when out_bf16."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    code = np.ascontiguousarray(code, dtype=np.float32)
    absmax = np.ascontiguousarray(absmax, dtype=np.float32)
    assert absmax.size == order * num_blocks(order, blocksize)
    if diag is not None:
        diag = np.ascontiguousarray(diag, dtype=np.float32)
    out = np.zeros((order, order), dtype=np.uint16 if out_bf16 else np.float32)
    rc = lib().qoracle_dequantize(_ptr(packed), _ptr(code), ct.c_int(order), ct.c_int(blocksize),
                                  ct.c_int(bits), _ptr(absmax), _ptr(diag), _ptr(out),
                                  ct.c_int(1 if out_bf16 else 0))
    if rc != 0:
        raise ValueError("qoracle_dequantize rejected its arguments")
    return out


def linear_map(signed=True, total_bits=4, power=2):
    """The reference's 'linear-2' codebook (qtensor/functional.py:106-113) as float32.

    Evenly spaced points on [-1, 1] (torch.linspace, so the fp32 bit patterns are the
    ones the reference gets), the entry at 2**(bits-1)-1 forced to 0, then sign*|x|**power.
    """
    import torch
    n = 2 ** total_bits
    if signed:
        pts = torch.linspace(-1, 1, n)
        pts[2 ** (total_bits - 1) - 1] = 0
    else:
        pts = torch.linspace(0, 1, n)
    return (pts.sign() * pts.abs().pow(power)).numpy().astype(np.float32)


def dynamic_map(signed=True, total_bits=4, power=1):
    """The reference's 'dynamic' codebook (qtensor/functional.py:87-103) as float32."""
    import torch
    vals = []
    ebits = total_bits - 1
    for i in range(ebits):
        items = int(2 ** i + 1 if signed else 2 ** (i + 1) + 1)
        edges = torch.linspace(0.1, 1, items)
        mids = (edges[:-1] + edges[1:]) / 2.0
        scale = 10 ** (-(ebits - 1) + i)
        vals += (scale * mids).tolist()
        if signed:
            vals += (-scale * mids).tolist()
    vals += [0, 1.0]
    vals.sort()
    t = torch.Tensor(vals)
    return (t.sign() * t.abs().pow(power)).numpy().astype(np.float32)
