"""Generates tests/golden/optimizer_cases.npz by running the REFERENCE optimizers on CPU.

    python tests/golden/make_optimizer_golden.py --ref /path/to/reference

The reference is imported, never copied or edited.  Three ways of running it:

  bits32     the reference as it runs on CPU: state silently forced to 32-bit
             (optimizers/shampoo2.py:134, shampoo1.py:128);
  bits4      4-bit state forced from outside by wrapping the module attributes
             QTensorSVDFast / QTensorDiagReal so they are built with bits=4; verbatim
             otherwise, so dequantize_blockwise_diagreal returns None
             (qtensor/functional.py:312-368) and the optimizers take their identity
             fallbacks (shampoo2.py:255-261);
  bits4_ret  as bits4, plus a wrapper around qtensor.functional.dequantize_blockwise_diagreal
             that returns the tensor the function fills.

Initial parameters and per-step gradients are shared by all cases (same seed) and stored
once; every case stores the parameters after each step.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# Square parameters and gradients with a well separated spectrum: on rank-deficient or
# near-degenerate statistics the reference's own result moves by 10-100 % of the update
# under a 1e-7 relative perturbation of the gradient (lower-half truncation picks among
# numerically tied Rayleigh quotients), so such inputs cannot pin anything.
SHAPES = [(64, 64), (80,), (72, 72), (16, 16, 1, 1), (1, 1, 40)]
HYPER = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=1, prec_maxorder=80,
             stat_decay=0.95, matrix_eps=1e-6, quan_blocksize=64)
STEPS = 2


def wellposed_grad(shape, g, lo=0.3):
    """U diag(s) W^T with s log-spaced in [lo, 1] (full rank, distinct singular values)."""
    dims = [d for d in shape if d != 1]
    if len(dims) < 2:
        return torch.randn(shape, generator=g) * 0.1
    rows = dims[0]
    cols = int(np.prod(shape)) // rows
    U, _ = torch.linalg.qr(torch.randn(rows, rows, generator=g, dtype=torch.float64))
    W, _ = torch.linalg.qr(torch.randn(cols, cols, generator=g, dtype=torch.float64))
    k = min(rows, cols)
    sv = torch.logspace(np.log10(lo), 0, k, dtype=torch.float64)
    return ((U[:, :k] * sv) @ W[:, :k].T).float().reshape(shape) * 0.1


def run_case(optim_cls, extra, seed, mode, modules):
    import qtensor.functional as RF
    undo = []
    if mode in ("bits4", "bits4_ret"):
        for mod in modules:
            for name in ("QTensorSVDFast", "QTensorDiagReal"):
                if hasattr(mod, name):
                    orig = getattr(mod, name)
                    setattr(mod, name, (lambda o: (lambda *a, **k: o(*a, **{**k, "bits": 4})))(orig))
                    undo.append((mod, name, orig))
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
        g = torch.Generator().manual_seed(seed)
        params = [torch.nn.Parameter(torch.randn(s, generator=g) * 0.5) for s in SHAPES]
        init = [p.detach().clone() for p in params]
        bits = 32 if mode == "bits32" else 4
        opt = optim_cls(params, prec_bits=bits, **HYPER, **extra)
        grads, after = [], []
        for step in range(STEPS):
            gs = [wellposed_grad(s, g) for s in SHAPES]
            for p, gr in zip(params, gs):
                p.grad = gr.clone()
            torch.manual_seed(1000 + step)          # PowerIter draws torch.rand
            opt.step()
            grads.append(gs)
            after.append([p.detach().clone() for p in params])
        return init, grads, after
    finally:
        for mod, name, orig in undo:
            setattr(mod, name, orig)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    cwd = os.getcwd()
    import tempfile
    os.chdir(tempfile.mkdtemp())                    # the reference writes logs/eigenvalues_*.csv
    import optimizers.shampoo1 as s1
    import optimizers.shampoo2 as s2

    cases = [
        ("s2_adamw", s2.ShampooAdamW, dict(rect_t1=1, rect_t2=4, inv_root_mode=0), [s2]),
        ("s2_adamw_newton", s2.ShampooAdamW, dict(rect_t1=1, rect_t2=4, inv_root_mode=1), [s2]),
        ("s2_sgd", s2.ShampooSGD, dict(momentum=0.9, nesterov=True), [s2]),
        ("s1_adamw", s1.ShampooAdamW, dict(), [s1]),
        ("s1_sgd", s1.ShampooSGD, dict(momentum=0.9), [s1]),
    ]
    blob, index = {}, []
    for name, cls, extra, mods in cases:
        for mode in ("bits32", "bits4", "bits4_ret"):
            if mode != "bits32" and name in ("s2_sgd", "s1_sgd"):
                continue
            init, grads, after = run_case(cls, extra, seed=11, mode=mode, modules=mods)
            key = f"{name}.{mode}"
            # every case starts from the same seed: parameters and gradients are stored once
            for i, t in enumerate(init):
                blob[f"init.{i}"] = t.numpy()
            for s in range(STEPS):
                for i in range(len(SHAPES)):
                    blob[f"grad.{s}.{i}"] = grads[s][i].numpy()
                    blob[f"{key}.after.{s}.{i}"] = after[s][i].numpy()
            index.append(dict(key=key, optimizer=name, mode=mode, extra=extra))
            print("done", key, flush=True)
    meta = dict(shapes=SHAPES, hyper=HYPER, steps=STEPS, cases=index)
    blob["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "optimizer_cases.npz"), **blob)


if __name__ == "__main__":
    main()
