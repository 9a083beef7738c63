"""Host logic of the optimizers on CPU with 32-bit state (the configuration in which the
reference itself runs on CPU), against parameters produced by the reference optimizers."""
import numpy as np
import pytest
import torch

from helpers import load_optimizer_cases, rel_fro

TOL = 1e-4      # relative Frobenius error of the post-step parameters


def build(optimizer, extra, hyper, params, bits):
    from optimizers import shampoo1, shampoo2
    mod = shampoo2 if optimizer.startswith("s2") else shampoo1
    cls = mod.ShampooAdamW if "adamw" in optimizer else mod.ShampooSGD
    return cls(params, prec_bits=bits, **hyper, **extra)


def run_case(blob, meta, case, device, bits):
    shapes = meta["shapes"]
    params = [torch.nn.Parameter(torch.from_numpy(blob[f"init.{i}"]).to(device)) for i in range(len(shapes))]
    opt = build(case["optimizer"], case["extra"], meta["hyper"], params, bits)
    errs, upd = [], []
    for s in range(meta["steps"]):
        before = [p.detach().cpu().numpy().copy() for p in params]
        for i, p in enumerate(params):
            p.grad = torch.from_numpy(blob[f"grad.{s}.{i}"]).to(device).clone()
        torch.manual_seed(1000 + s)
        opt.step()
        got = [p.detach().cpu().numpy() for p in params]
        want = [blob[f"{case['key']}.after.{s}.{i}"] for i in range(len(shapes))]
        errs.append(rel_fro(got, want))
        # error relative to the size of the update itself (much stricter than the parameter norm)
        upd.append(rel_fro([g - b for g, b in zip(got, before)], [w - b for w, b in zip(want, before)]))
    return errs, upd


def cases(mode):
    _, meta = load_optimizer_cases()
    return [c for c in meta["cases"] if c["mode"] == mode]


@pytest.mark.parametrize("case", cases("bits32"), ids=lambda c: c["key"])
def test_cpu_32bit_step_matches_reference(case):
    blob, meta = load_optimizer_cases()
    errs, upd = run_case(blob, meta, case, "cpu", 32)
    assert max(errs) < TOL, errs
    # the Schur-Newton variants draw their power-iteration start from the global RNG in a
    # different order than the reference (batched), which moves the ridge slightly
    loose = "newton" in case["key"] or case["key"].startswith("s1")
    assert max(upd) < (5e-2 if loose else 1e-3), upd


def test_lowbit_on_cpu_is_refused():
    from optimizers.shampoo2 import ShampooAdamW
    p = torch.nn.Parameter(torch.randn(80, 80))
    p.grad = torch.randn(80, 80)
    opt = ShampooAdamW([p], prec_bits=4)
    with pytest.raises(RuntimeError):
        opt.step()


def test_block_partitioner_roundtrip():
    from optimizers.shampoo2 import BlockPartitioner
    t = torch.arange(7 * 10, dtype=torch.float32).reshape(7, 10)
    bp = BlockPartitioner(t, 4)
    assert bp.shapes_for_preconditioners() == [[4, 4], [4, 4], [4, 4], [4, 4], [4, 4], [2, 2],
                                               [3, 3], [4, 4], [3, 3], [4, 4], [3, 3], [2, 2]]
    parts = bp.partition(t)
    assert [tuple(p.shape) for p in parts] == [(4, 4), (4, 4), (4, 2), (3, 4), (3, 4), (3, 2)]
    assert torch.equal(bp.merge_partitions(parts), t)
    assert bp.num_splits() == 2
    # a dimension that is an exact multiple makes no empty block (reference: (d-1)//block_size)
    assert [tuple(p.shape) for p in BlockPartitioner(torch.zeros(8, 3), 4).partition(torch.zeros(8, 3))] == [(4, 3), (4, 3)]
    # merge: every split pattern (none, rows only, columns only, both), with and without a destination
    for shape in ((3, 4), (10, 3), (3, 10), (7, 10)):
        x = torch.randn(*shape)
        q = BlockPartitioner(x, 4)
        blocks = [b.clone() for b in q.partition(x)]
        assert torch.equal(q.merge_partitions(blocks), x)
        dst = torch.full(shape, 7.0)
        got = q.merge_partitions(blocks, out=dst)
        assert got.data_ptr() == dst.data_ptr() and torch.equal(dst, x)


def test_ridged_inverse_root_equals_reference_where_it_is_finite():
    """(S + rho)^(-1/p) of the reference (functional.py:760-762) wherever S + rho > 0; a Rayleigh
    quotient that rounding pushed to or below -rho (the reference returns inf / NaN there) counts
    as the zero it stands for."""
    import qtensor.functional as F
    S = torch.tensor([[2.0, 0.5, 0.0, -5e-7, -1e-6, -1.0025e-6, -3e-6]])
    rho = torch.tensor([[1e-6]])
    got = F.ridged_inverse_root(S, rho, 4)
    want = 1 / (S + rho).pow(0.25)
    finite = torch.isfinite(want)
    assert finite.tolist() == [[True, True, True, True, False, False, False]]
    assert torch.equal(got[finite], want[finite])
    assert torch.equal(got[~finite], (1 / rho.pow(0.25)).expand_as(S)[~finite])
    assert torch.isfinite(got).all()
    # scalar ridge, as the single-matrix form passes it
    assert torch.equal(F.ridged_inverse_root(S[0], 1e-6 * torch.tensor(1.0), 4), got[0])
