"""Generates tests/golden/quant_cases.npz by running the REFERENCE's own CPU quantizer.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py --ref /path/to/reference

The reference (qtensor/functional.py) is imported, never copied.  Every case stores its
inputs and the reference's outputs, so the fixtures are self-contained on machines
where the reference is absent.  bf16 tensors are stored as uint16 bit patterns.
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def spd_logspectrum(n, seed):
    """Q diag(lambda) Q^T with Q from the QR of a seeded N(0,1) matrix, lambda log-uniform in [1e-6, 1]."""
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=g))
    lam = torch.exp(torch.empty(n, dtype=torch.float64).uniform_(np.log(1e-6), 0.0, generator=g))
    a = (q * lam) @ q.T
    return (0.5 * (a + a.T)).float()


def bf16_bits(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    import qtensor.functional as RF

    codes = {
        "linear4": RF.create_linear_map(True, 4, 2),
        "linear8": RF.create_linear_map(True, 8, 2),
        "dynamic4": RF.create_dynamic_map(True, 4, 1),
    }
    g = torch.Generator().manual_seed(1234)
    perm = torch.randperm(16, generator=g)
    codes["shuffled4"] = codes["linear4"][perm].clone()

    def randn(n, scale=1.0):
        return torch.randn(n, n, generator=g) * scale

    def wide(n):
        """columns spanning eight decades, a zero row segment and exact +-absmax ties."""
        a = randn(n)
        a *= torch.logspace(-6, 2, n).unsqueeze(0)
        if n > 70:
            a[3, 64:] = 0.0
        a[1, :] = a[1, 0]
        return a

    cases = []   # (name, A, code_name, order, blocksize, bits, diagreal, in_bf16, out_bf16)
    cases.append(("kat8", randn(8), "linear4", 8, 64, 4, False, False, False))
    cases.append(("n64", randn(64), "linear4", 64, 64, 4, False, False, False))
    cases.append(("n65_odd", randn(65), "linear4", 65, 64, 4, False, False, False))
    cases.append(("n65_odd_diag", randn(65), "linear4", 65, 64, 4, True, False, False))
    cases.append(("n100_tail", wide(100), "linear4", 100, 64, 4, False, False, False))
    cases.append(("n100_tail_diag", wide(100), "linear4", 100, 64, 4, True, False, False))
    cases.append(("eye128", torch.eye(128), "linear4", 128, 64, 4, False, False, False))
    cases.append(("eye128_diag", torch.eye(128), "linear4", 128, 64, 4, True, False, False))
    cases.append(("eps_eye96", 1e-6 * torch.eye(96), "linear4", 96, 64, 4, False, False, False))
    cases.append(("n130_bs128", wide(130), "linear4", 130, 128, 4, False, False, False))
    cases.append(("n200_bs256", randn(200, 1e-3), "linear4", 200, 256, 4, True, False, False))
    cases.append(("n96_8bit", wide(96), "linear8", 96, 64, 8, False, False, False))
    cases.append(("n96_8bit_diag", wide(96), "linear8", 96, 64, 8, True, False, False))
    cases.append(("n72_dynamic", randn(72), "dynamic4", 72, 64, 4, False, False, False))
    cases.append(("n72_shuffled", randn(72), "shuffled4", 72, 64, 4, True, False, False))
    cases.append(("n80_bf16", randn(80).bfloat16(), "linear4", 80, 64, 4, False, True, True))
    cases.append(("n80_bf16_diag", randn(80).bfloat16(), "linear4", 80, 64, 4, True, True, True))
    cases.append(("spd256", spd_logspectrum(256, 7), "linear4", 256, 64, 4, False, False, False))
    cases.append(("spd256_diag", spd_logspectrum(256, 7), "linear4", 256, 64, 4, True, False, False))

    blob = {}
    index = []
    for name, A, cname, n, bs, bits, dr, in_bf16, out_bf16 in cases:
        code = codes[cname]
        outdtype = torch.bfloat16 if out_bf16 else torch.float32
        if dr:
            q, am, dg = RF.quantize_blockwise_diagreal(A, code, n, blocksize=bs, bits=bits)
            # the public diagreal dequantizer of the reference returns None (it lacks a
            # return statement); its CPU worker fills and returns the tensor.
            d = RF._dequantize_blockwise_cpu(q, code, n, am, None, bs, bits, outdtype, diag=dg)
            blob[name + ".diag"] = dg.numpy().copy()
        else:
            q, am = RF.quantize_blockwise(A, code, n, blocksize=bs, bits=bits)
            d = RF.dequantize_blockwise(q, code, n, am, outdtype=outdtype, blocksize=bs, bits=bits)
        # the reference's vectorised variant agrees with its loop variant for plain
        # (non-diagreal; its diagreal branch does not zero the diagonal) [-1,1] codebooks
        if not dr and cname.startswith("linear"):
            qv = RF._quantize_blockwise_vectorized(A, code, n, None, None, bs, bits)
            assert torch.equal(qv[0], q) and torch.equal(qv[1], am), name
        blob[name + ".A"] = bf16_bits(A) if in_bf16 else A.numpy().copy()
        blob[name + ".packed"] = q.numpy().copy()
        blob[name + ".absmax"] = am.numpy().copy()
        blob[name + ".deq"] = bf16_bits(d) if out_bf16 else d.numpy().copy()
        index.append(dict(name=name, code=cname, order=n, blocksize=bs, bits=bits, diagreal=dr,
                          in_bf16=in_bf16, out_bf16=out_bf16))
    for k, v in codes.items():
        blob["code." + k] = v.numpy().copy()
    blob["index"] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **blob)

    # Config-1 matrix (1024 x 1024 SPD, seed 0): too large to commit; record hashes instead.
    A = spd_logspectrum(1024, 0)
    code = codes["linear4"]
    q, am = RF.quantize_blockwise(A, code, 1024, blocksize=64, bits=4)
    d = RF.dequantize_blockwise(q, code, 1024, am, blocksize=64, bits=4)
    qd, amd, dg = RF.quantize_blockwise_diagreal(A, code, 1024, blocksize=64, bits=4)
    sha = lambda t: hashlib.sha256(t.numpy().tobytes()).hexdigest()
    rec = dict(seed=0, order=1024, blocksize=64, bits=4,
               input_sha256=sha(A), packed_sha256=sha(q), absmax_sha256=sha(am), deq_sha256=sha(d),
               diag_packed_sha256=sha(qd), diag_absmax_sha256=sha(amd), diag_sha256=sha(dg),
               roundtrip_rel_fro=float((d - A).norm() / A.norm()))
    with open(os.path.join(HERE, "config1_hashes.json"), "w") as f:
        json.dump(rec, f, indent=1)
    print("wrote", len(cases), "cases;", rec)


if __name__ == "__main__":
    main()
