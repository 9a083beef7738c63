"""Parity of the optimizer step at the preconditioner orders the headline benchmark runs on
(672 .. 1200, ViT-B/32) and at the orders of the ResNet-34 and Swin-Tiny configurations.

Three layers of evidence:
  1. tests/golden/large_order_cases.npz - parameters produced by the REFERENCE shampoo2-AdamW
     (CPU, 4-bit forced) on 768 x 768 and 1200 x 1200 parameters.  The CPU oracle is checked
     against it here without a GPU, the CUDA path with one (eager and CUDA-graph replay).
  2. CUDA path against the oracle run on the fly, per matrix: the dequantized 4-bit
     preconditioner P = L^(-1/4), the preconditioned block P_L G P_R, and the parameters.
  3. The real (non-square) shapes of one ViT-B/32 encoder layer and of ResNet-34 / Swin-Tiny
     layers.  Their statistics are rank-deficient by construction (G G^T of a 1200 x 768
     block has rank <= 768), and there the reference's own result is not a function of its
     inputs to better than the 4-bit quantisation noise: the basis of the null space comes
     out of rounding noise in the QR, and a different basis quantises to different codes.  The
     bound used for those cases is stated next to each assertion.

Tolerance on post-step parameters: 1e-4 relative Frobenius error - or, where that is larger,
YARD_FACTOR times the SENSITIVITY YARDSTICK of the case.  The yardstick is how far the reference's
own fp32 result is from (a) the same computation with one fp32 rounding of the statistics update
evaluated in another order (OracleShampoo(alternate_rounding=True)) and (b) the same
computation with every product and the QR in float64 (wide_arithmetic=True), whichever is
larger.  The step amplifies rounding through 4-bit codes that flip: a relative change of
1e-6 in an eigenvector matrix moves one code in 10^5 across a decision threshold, and each flip
moves that element by a whole code step.  At order 1200 the float64 twin ends 1.3e-3 away from
the fp32 oracle in the parameters (109-157 code bytes of the stored eigenbasis differ), at order
768 1.8e-4, at order 672 5e-6: no implementation, the reference's own CUDA path included, can
agree with the CPU reference more closely than that on such a case, and the 1e-4 of the small
orders is out of reach there for reasons that are the algorithm's, not the kernels'.

Intermediates (the dequantized 4-bit preconditioner, the preconditioned block) are compared
AFTER quantization, where the same effect is at its strongest; FLIP_BOUND states the distance
a handful of differing codes makes.  The CUDA path multiplies from scaled fp16 operand planes
(22 significant bits) with 128-k accumulation chains; measured against the oracle it sits at the
yardstick itself (order 768: preconditioners 2.6e-4 / 2.1e-4 with a yardstick of 2.3e-4, parameters
1.3e-4 with 1.8e-4; order 1200: 1.4e-3 / 2.2e-3 with 2.1e-3, parameters 1.1e-3 with 1.3e-3; order
336: 8e-7).  With bf16 operand planes (16 bits) the same cases were 4 to 7 times further away."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import GOLDEN, hashed_matrix, wellposed_matrix

TOL = 1e-4
YARD_FACTOR = 5.0       # headroom over the reference's own fp32-evaluation sensitivity (two independent roundings + margin)
FLIP_BOUND = 2.5e-3     # 4-bit results compared after quantization at orders >= 336 (see the module docstring)
ONE_FLIP = 1e-3         # parameters of an n x n block, n >= 336: what ONE differing code of the stored eigenbasis
                        # (1 in ~3e5) does to them through the AdamW step (measured 4e-6 .. 6e-4 over variants of the arithmetic: one or two flips)


def load_large():
    blob = np.load(os.path.join(GOLDEN, "large_order_cases.npz"))
    meta = json.loads(bytes(blob["meta"]).decode())
    return blob, meta


def large_inputs(meta):
    shapes = [tuple(s) for s in meta["shapes"]]
    init = [torch.from_numpy(hashed_matrix(s, seed, meta["init_scale"])) for s, seed in zip(shapes, meta["init_seeds"])]
    grads = [[torch.from_numpy(wellposed_matrix(s, seed, meta["grad_scale"])) for s, seed in zip(shapes, row)]
             for row in meta["grad_seeds"]]
    return shapes, init, grads


def hyper_of(meta):
    h = dict(meta["hyper"])
    h["betas"] = tuple(h["betas"])
    return h


def sample_errors(blob, meta, mode, t, params, init):
    """(parameter error, update error) of `params` against the stored sample of the reference's
    parameters after step t; both relative Frobenius over the sampled elements of all tensors."""
    stride = meta["stride"]
    num = den = upd = 0.0
    for i, p in enumerate(params):
        got = np.asarray(p, dtype=np.float64).reshape(-1)[::stride]
        want = blob[f"{mode}.after.{t}.{i}.sample"].astype(np.float64)
        prev = (blob[f"{mode}.after.{t - 1}.{i}.sample"] if t > 0 else init[i].numpy().reshape(-1)[::stride]).astype(np.float64)
        num += float(((got - want) ** 2).sum())
        den += float((want ** 2).sum())
        upd += float(((want - prev) ** 2).sum())
    return (num / den) ** 0.5, (num / upd) ** 0.5


# --------------------------------------------------------------------------------------
# 1. reference fixtures at orders 768 and 1200
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode", ["bits4_ret", "bits4"])
def test_oracle_matches_reference_at_orders_768_and_1200(mode):
    """Pins the CPU oracle at large order: same inputs, parameters within 1e-4 of the reference's."""
    from oracle.shampoo_oracle import OracleShampoo
    blob, meta = load_large()
    shapes, init, grads = large_inputs(meta)
    params = [t.clone() for t in init]
    h = hyper_of(meta)
    opt = OracleShampoo(params, kind="adamw", flavour="s2", prec_bits=4, diagreal_none=(mode == "bits4"), **h)
    for t in range(meta["steps"]):
        opt.step([g.clone() for g in grads[t]])
        perr, uerr = sample_errors(blob, meta, mode, t, [p.numpy() for p in params], init)
        print(mode, "step", t, "param err", perr, "update err", uerr)
        assert perr < TOL, (mode, t, perr, uerr)


@pytest.mark.gpu
@pytest.mark.parametrize("graph", [False, True], ids=["eager", "graph"])
@pytest.mark.parametrize("mode", ["bits4_ret", "bits4"])
def test_cuda_step_matches_reference_at_orders_768_and_1200(native_lib, mode, graph):
    from optimizers import _engine
    from optimizers.shampoo2 import ShampooAdamW
    from oracle.shampoo_oracle import OracleShampoo
    blob, meta = load_large()
    shapes, init, grads = large_inputs(meta)
    ps = [torch.nn.Parameter(t.clone().cuda()) for t in init]
    alt = [t.clone() for t in init]
    wide = [t.clone() for t in init]
    ora_alt = OracleShampoo(alt, kind="adamw", flavour="s2", prec_bits=4, diagreal_none=(mode == "bits4"),
                            alternate_rounding=True, **hyper_of(meta))
    ora_wide = OracleShampoo(wide, kind="adamw", flavour="s2", prec_bits=4, diagreal_none=(mode == "bits4"),
                             wide_arithmetic=True, **hyper_of(meta))
    _engine.REFERENCE_DIAGREAL_NONE = (mode == "bits4")
    try:
        opt = ShampooAdamW(ps, prec_bits=4, cuda_graph=graph, **hyper_of(meta))
        for t in range(meta["steps"]):
            for p, g in zip(ps, grads[t]):
                p.grad = g.clone().cuda()
            opt.step()
            torch.cuda.synchronize()
            ora_alt.step([g.clone() for g in grads[t]])
            ora_wide.step([g.clone() for g in grads[t]])
            yard = max(sample_errors(blob, meta, mode, t, [p.numpy() for p in alt], init)[0],
                       sample_errors(blob, meta, mode, t, [p.numpy() for p in wide], init)[0])
            perr, uerr = sample_errors(blob, meta, mode, t, [p.detach().cpu().numpy() for p in ps], init)
            print(mode, "graph" if graph else "eager", "step", t, "param err", perr, "update err", uerr, "yardstick", yard)
            assert perr < max(TOL, YARD_FACTOR * yard), (mode, t, perr, uerr, yard)
    finally:
        _engine.REFERENCE_DIAGREAL_NONE = False
    assert native_lib.qt_device_error(1) == 0


# --------------------------------------------------------------------------------------
# 2. per-matrix intermediates against the oracle, square blocks of every model order
# --------------------------------------------------------------------------------------
HEADLINE_HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05, stat_compute_steps=1,
                      prec_compute_steps=1, prec_maxorder=1200, stat_decay=0.95, matrix_eps=1e-6, quan_blocksize=64,
                      rect_t1=1, rect_t2=4, inv_root_mode=0)


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


class Run:
    """Steps the CUDA optimizer, the CPU oracle and the oracle's alternate-rounding twin on the
    same deterministic inputs."""

    def __init__(self, shapes, steps, seed, hyper=HEADLINE_HYPER, graph=False, cuda=True):
        from oracle.shampoo_oracle import OracleShampoo
        self.shapes = shapes
        init = [torch.from_numpy(hashed_matrix(s, seed + i, 2.0 ** -5)) for i, s in enumerate(shapes)]
        self.ref = [t.clone() for t in init]
        self.alt = [t.clone() for t in init]
        self.wide = [t.clone() for t in init]
        self.ora = OracleShampoo(self.ref, kind="adamw", flavour="s2", prec_bits=4, **hyper)
        self.ora_alt = OracleShampoo(self.alt, kind="adamw", flavour="s2", prec_bits=4, alternate_rounding=True, **hyper)
        self.ora_wide = OracleShampoo(self.wide, kind="adamw", flavour="s2", prec_bits=4, wide_arithmetic=True, **hyper)
        self.ps = self.opt = None
        if cuda:
            from optimizers.shampoo2 import ShampooAdamW
            self.ps = [torch.nn.Parameter(t.clone().cuda()) for t in init]
            self.opt = ShampooAdamW(self.ps, prec_bits=4, cuda_graph=graph, **hyper)
        for t in range(steps):
            self.grads = [torch.from_numpy(wellposed_matrix(s, seed + 100 * (t + 1) + i)) for i, s in enumerate(shapes)]
            if cuda:
                for p, g in zip(self.ps, self.grads):
                    p.grad = g.clone().cuda()
                self.opt.step()
            self.ora.step([g.clone() for g in self.grads])
            self.ora_alt.step([g.clone() for g in self.grads])
            self.ora_wide.step([g.clone() for g in self.grads])
        if cuda:
            torch.cuda.synchronize()

    def yardstick(self, i):
        return max(rel(self.alt[i].numpy(), self.ref[i].numpy()), rel(self.wide[i].numpy(), self.ref[i].numpy()))

    def tolerance(self, i):
        """max(1e-4, YARD_FACTOR x yardstick) for the parameters of tensor i; tensors with
        preconditioner orders of 336 and more get at least ONE_FLIP (see its definition)."""
        dims = [d for d in self.shapes[i] if d != 1]
        big = len(dims) >= 2 and max(dims[0], int(np.prod(dims[1:]))) >= 336
        return max(TOL, YARD_FACTOR * self.yardstick(i), ONE_FLIP if big else 0.0)

    def param_error(self, i):
        return rel(self.ps[i].detach().cpu().numpy(), self.ref[i].numpy())


@pytest.mark.gpu
@pytest.mark.parametrize("n", [672, 768, 1000, 1104, 1200, 100, 336, 576, 1008, 1152])
def test_square_block_intermediates_match_oracle(native_lib, n):
    """One n x n parameter, two steps: the dequantized 4-bit preconditioners, the preconditioned
    gradient block and the parameters against the oracle's."""
    r = Run([(n, n)], 2, seed=7 * n)
    pre = r.opt.state[r.ps[0]]["preconditioner"]
    st, st_alt, st_wide = r.ora.state[0], r.ora_alt.state[0], r.ora_wide.state[0]
    flip = FLIP_BOUND if n >= 336 else TOL
    for axis in range(2):
        P_gpu = pre.preconditioners[axis].dequantize().cpu().numpy()
        P_ref = st.precs[axis].load().numpy()
        yard = max(rel(st_alt.precs[axis].load().numpy(), P_ref), rel(st_wide.precs[axis].load().numpy(), P_ref))
        e = rel(P_gpu, P_ref)
        print(f"order {n} axis {axis}: preconditioner error {e:.3e} (yardstick {yard:.3e})")
        assert e < max(flip, YARD_FACTOR * yard), (n, axis, e, yard)
    g = r.grads[0]
    blk_ref = r.ora._preconditioned(st, g.clone()).numpy()
    yard = max(rel(r.ora_alt._preconditioned(st_alt, g.clone()).numpy(), blk_ref),
               rel(r.ora_wide._preconditioned(st_wide, g.clone()).numpy(), blk_ref))
    e = rel(pre.preconditioned_grad(g.cuda()).cpu().numpy(), blk_ref)
    print(f"order {n}: preconditioned block error {e:.3e} (yardstick {yard:.3e})")
    assert e < max(flip, YARD_FACTOR * yard), (n, e, yard)
    e = r.param_error(0)
    print(f"order {n}: parameter error {e:.3e} (tolerance {r.tolerance(0):.3e})")
    assert e < r.tolerance(0), (n, e)
    assert native_lib.qt_device_error(1) == 0


# --------------------------------------------------------------------------------------
# 3. real layer shapes (rank-deficient statistics)
# --------------------------------------------------------------------------------------
VIT_LAYER = [(2304, 768), (2304,), (768, 768), (768,), (3072, 768), (3072,), (768, 3072), (768,)]
RESNET_SUBSET = [(64, 3, 3, 3), (64, 64, 3, 3), (128, 64, 1, 1), (128, 128, 3, 3), (256, 256, 3, 3), (512, 512, 3, 3),
                 (100, 512), (100,)]
SWIN_SUBSET = [(96, 3, 2, 2), (49, 3), (49, 6), (9, 24), (288, 96), (96, 384), (192, 384), (576, 192), (384, 1536), (1152, 384),
               (768, 3072), (2304, 768), (100, 768)]



@pytest.mark.gpu
@pytest.mark.parametrize("graph", [False, True], ids=["eager", "graph"])
def test_vit_encoder_layer_step(native_lib, graph):
    """qkv, proj, fc1, fc2 of one ViT-B/32 encoder layer (orders 672, 768, 1104, 1200), two steps,
    T1 = T2 = 1, eager and replayed as a CUDA graph."""
    r = Run(VIT_LAYER, 2, seed=31, graph=graph)
    for i, s in enumerate(VIT_LAYER):
        e = r.param_error(i)
        print("vit layer", s, "graph" if graph else "eager", f"parameter error {e:.3e} (tolerance {r.tolerance(i):.3e})")
        assert e < r.tolerance(i), (s, e, r.tolerance(i))
    assert native_lib.qt_device_error(1) == 0


@pytest.mark.gpu
def test_vit_encoder_layer_graph_replay_equals_eager(native_lib):
    a = Run(VIT_LAYER, 3, seed=31, graph=False)
    b = Run(VIT_LAYER, 3, seed=31, graph=True)
    assert b.opt._use_graph and b.opt._graph_state is not None
    for s, x, y in zip(VIT_LAYER, a.ps, b.ps):
        e = rel(y.detach().cpu().numpy(), x.detach().cpu().numpy())
        assert e < 1e-5, (s, e)


@pytest.mark.gpu
@pytest.mark.parametrize("name,shapes", [("resnet34", RESNET_SUBSET), ("swin_tiny", SWIN_SUBSET)])
def test_model_subsets_cover_every_order(native_lib, name, shapes):
    """One step on a subset of each model's parameter shapes that contains every distinct
    preconditioner order of the model (100, 336, 576, 1008, 1152, ... and the small fp32 ones)."""
    import workloads
    model = workloads.resnet34_cifar() if name == "resnet34" else workloads.swin_tiny_32()
    full = workloads.preconditioner_census([tuple(p.shape) for p in model.parameters()])
    assert set(workloads.preconditioner_census(shapes)) == set(full), "subset misses an order of the model"
    r = Run(shapes, 1, seed=57)
    for i, s in enumerate(shapes):
        e = r.param_error(i)
        print(name, s, f"parameter error {e:.3e} (tolerance {r.tolerance(i):.3e})")
        assert e < r.tolerance(i), (s, e, r.tolerance(i))
    assert native_lib.qt_device_error(1) == 0
