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
