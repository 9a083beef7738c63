"""Generates tests/golden/large_order_cases.npz by running the REFERENCE shampoo2-AdamW on CPU
with 4-bit state at the preconditioner orders of the ViT-B/32 step (768 and 1200).

    python tests/golden/make_large_order_golden.py --ref /path/to/reference

The reference is imported, never copied or edited; 4-bit state is forced from outside and its
dequantize_blockwise_diagreal is wrapped so that it returns the tensor it fills (the modes
"bits4" and "bits4_ret" of make_optimizer_golden.py).  Inputs are NOT stored: initial parameters
and gradients come from tests/helpers.py (hashed_matrix, wellposed_matrix: integer arithmetic and
single correctly-rounded fp32 operations, bit-identical everywhere; the gradients are well
conditioned on purpose - on a generic dense matrix the reference's step amplifies a 1e-7
rounding difference to 1e-2 of the update, which nothing can be pinned against), so the file
holds only the recipe and, per step and parameter, a strided sample
of the reference's post-step parameters plus the norms needed for relative errors.
Takes a few minutes (the reference's CPU quantizer is a Python loop over row blocks).
"""
import argparse
import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from helpers import hashed_matrix, wellposed_matrix  # noqa: E402

SHAPES = [(768, 768), (768,), (1200, 1200)]
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=1,
             prec_maxorder=1200, stat_decay=0.95, matrix_eps=1e-6, quan_blocksize=64, rect_t1=1, rect_t2=4,
             inv_root_mode=0)
STEPS = 2
STRIDE = 41                      # sample every 41st element of the flat parameter
INIT_SCALE, GRAD_SCALE = 2.0 ** -5, 2.0 ** -4


def inputs():
    init = [torch.from_numpy(hashed_matrix(s, 100 + i, INIT_SCALE)) for i, s in enumerate(SHAPES)]
    grads = [[torch.from_numpy(wellposed_matrix(s, 1000 + 10 * t + i, GRAD_SCALE)) for i, s in enumerate(SHAPES)]
             for t in range(STEPS)]
    return init, grads


def run(mode):
    import optimizers.shampoo2 as s2
    import qtensor.functional as RF
    undo = []
    for name in ("QTensorSVDFast", "QTensorDiagReal"):
        orig = getattr(s2, name)
        setattr(s2, name, (lambda o: (lambda *a, **k: o(*a, **{**k, "bits": 4})))(orig))
        undo.append((s2, name, orig))
    if mode == "bits4_ret":
        orig_fn = RF.dequantize_blockwise_diagreal

        def with_return(A, code, order, absmax, diag, outdtype=torch.float32, out=None, blocksize=256, bits=8):
            if out is None:
                out = torch.empty((order, order), dtype=outdtype, device=A.device)
            orig_fn(A, code, order, absmax, diag, outdtype=outdtype, out=out, blocksize=blocksize, bits=bits)
            return out
        RF.dequantize_blockwise_diagreal = with_return
        undo.append((RF, "dequantize_blockwise_diagreal", orig_fn))
    try:
        init, grads = inputs()
        params = [torch.nn.Parameter(t.clone()) for t in init]
        opt = s2.ShampooAdamW(params, prec_bits=4, **HYPER)
        after = []
        for t in range(STEPS):
            for p, g in zip(params, grads[t]):
                p.grad = g.clone()
            opt.step()
            after.append([p.detach().clone() for p in params])
            print(mode, "step", t, "done", flush=True)
        return init, after
    finally:
        for mod, name, orig in undo:
            setattr(mod, name, orig)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    cwd = os.getcwd()
    os.chdir(tempfile.mkdtemp())                    # the reference writes logs/eigenvalues_*.csv
    blob = {}
    for mode in ("bits4_ret", "bits4"):
        init, after = run(mode)
        prev = init
        for t in range(STEPS):
            for i, a in enumerate(after[t]):
                flat = a.numpy().reshape(-1)
                blob[f"{mode}.after.{t}.{i}.sample"] = flat[::STRIDE].copy()
                blob[f"{mode}.after.{t}.{i}.norm"] = np.float64(np.linalg.norm(flat.astype(np.float64)))
                blob[f"{mode}.update.{t}.{i}.norm"] = np.float64(
                    np.linalg.norm((a - prev[i]).numpy().astype(np.float64).reshape(-1)))
            prev = after[t]
    meta = dict(shapes=SHAPES, hyper={k: (list(v) if isinstance(v, tuple) else v) for k, v in HYPER.items()},
                steps=STEPS, stride=STRIDE, init_scale=INIT_SCALE, grad_scale=GRAD_SCALE,
                init_seeds=[100 + i for i in range(len(SHAPES))],
                grad_seeds=[[1000 + 10 * t + i for i in range(len(SHAPES))] for t in range(STEPS)],
                modes=["bits4_ret", "bits4"])
    blob["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "large_order_cases.npz"), **blob)
    print("wrote", os.path.join(HERE, "large_order_cases.npz"))


if __name__ == "__main__":
    main()
