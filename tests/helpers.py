"""Shared helpers of the test suite: golden-fixture access and input generators."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")


def load_quant_cases():
    blob = np.load(os.path.join(GOLDEN, "quant_cases.npz"))
    index = json.loads(bytes(blob["index"]).decode())
    return blob, index


def case_ids():
    _, index = load_quant_cases()
    return [c["name"] for c in index]


def spd_logspectrum(n, seed):
    """Q diag(lambda) Q^T, Q from the QR of a seeded N(0,1) matrix, lambda log-uniform in [1e-6, 1]
    (the construction of the 1024 x 1024 round-trip configuration)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g))
    lam = torch.exp(torch.empty(n, dtype=torch.float64).uniform_(np.log(1e-6), 0.0, generator=g))
    a = (q * lam) @ q.T
    return (0.5 * (a + a.T)).float()


def bits_equal(a, b):
    """Bit-pattern equality of two arrays of the same dtype and shape (distinguishes -0.0 from +0.0)."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return a.tobytes() == b.tobytes()


def load_optimizer_cases():
    blob = np.load(os.path.join(GOLDEN, "optimizer_cases.npz"))
    meta = json.loads(bytes(blob["meta"]).decode())
    return blob, meta


def rel_fro(a, b):
    """Relative Frobenius error ||a-b|| / ||b|| over a list of arrays taken as one vector."""
    num = sum(float(np.sum((np.asarray(x, dtype=np.float64) - np.asarray(y, dtype=np.float64)) ** 2)) for x, y in zip(a, b))
    den = sum(float(np.sum(np.asarray(y, dtype=np.float64) ** 2)) for y in b)
    return (num / max(den, 1e-300)) ** 0.5


def hashed_matrix(shape, seed, scale=1.0):
    """Pseudo-random fp32 array with entries in [-scale, scale), computed in 64-bit integer
    arithmetic only (a splitmix64 finaliser of the flat index), then one exact int -> float
    conversion and a multiplication by `scale` (use a power of two).  Bit-identical on every
    machine, so large inputs of golden cases need not be stored: only (shape, seed, scale) is."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        z = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    v = (z >> np.uint64(40)).astype(np.int64) - (1 << 23)          # 24-bit signed integers
    return (v.astype(np.float32) * np.float32(scale / (1 << 23))).reshape(shape)


def _hash64(n, seed):
    with np.errstate(over="ignore"):
        z = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def wellposed_matrix(shape, seed, scale=2.0 ** -4):
    """Gradient-like fp32 array whose (rows x cols) matrix form - rows = first non-unit dimension -
    is well conditioned: a shuffled 'diagonal' of min(rows, cols) distinct values spaced linearly
    in [0.3, 1] plus dense hashed noise of amplitude 2^-9 (spectral norm below 0.1), all times
    `scale`.  Its singular values stay within about 0.1 of the diagonal values, so G G^T and
    G^T G have a condition number near 10 on their range and well separated eigenvalues; the
    reference's own step is then insensitive to rounding (measured: its parameters move by
    5e-6 relative between two fp32 evaluation orders, against 1e-2 for a generic dense matrix
    whose smallest singular values fall below the 1e-6 ridge).  Every element is produced by
    integer arithmetic and single correctly-rounded fp32 operations: bit-identical everywhere.
    Vectors (fewer than two non-unit dimensions) are plain hashed noise."""
    dims = [d for d in shape if d != 1]
    if len(dims) < 2:
        return hashed_matrix(shape, seed, scale)
    rows = dims[0]
    cols = int(np.prod(shape)) // rows
    k = min(rows, cols)
    G = hashed_matrix((rows, cols), seed, 2.0 ** -9)
    perm = np.argsort(_hash64(k, seed + 7919), kind="stable").astype(np.float32)
    d = np.float32(0.3) + np.float32(0.7) * perm / np.float32(max(k - 1, 1))
    idx = np.arange(k)
    G[idx, idx] = G[idx, idx] + d
    return (G * np.float32(scale)).reshape(shape)
