"""Checkpoint / resume: optimizer.state_dict() -> torch.save -> load_state_dict() in a fresh
optimizer continues exactly where the uninterrupted run would be (the reference saves the same
objects, train_cifar.py:446-460, and re-homes them in load_state_dict, shampoo2.py:311-317)."""
import io

import pytest
import torch

SHAPES_CPU = [(40, 24), (24,), (56, 56)]
SHAPES_GPU = [(128, 96), (96,), (80, 80)]


def _roundtrip(device, shapes, hyper, steps=6, cut=3):
    from optimizers.shampoo2 import ShampooAdamW

    def make():
        g = torch.Generator().manual_seed(1)
        ps = [torch.nn.Parameter(torch.randn(s, generator=g).to(device)) for s in shapes]
        return ps, ShampooAdamW(ps, **hyper)

    g = torch.Generator().manual_seed(2)
    grads = [[(torch.randn(s, generator=g) * 0.1).to(device) for s in shapes] for _ in range(steps)]

    def advance(ps, opt, lo, hi):
        for t in range(lo, hi):
            for p, gr in zip(ps, grads[t]):
                p.grad = gr.clone()
            opt.step()

    ps, opt = make()
    advance(ps, opt, 0, steps)
    want = [p.detach().cpu().clone() for p in ps]

    ps, opt = make()
    advance(ps, opt, 0, cut)
    buf = io.BytesIO()
    torch.save({"opt": opt.state_dict(), "params": [p.detach().cpu() for p in ps]}, buf)
    buf.seek(0)
    ck = torch.load(buf, weights_only=False)
    ps2, opt2 = make()
    for p, q in zip(ps2, ck["params"]):
        p.data.copy_(q)
    opt2.load_state_dict(ck["opt"])
    advance(ps2, opt2, cut, steps)
    got = [p.detach().cpu() for p in ps2]
    return max(float((a - b).abs().max()) for a, b in zip(got, want))


def test_resume_cpu_32bit():
    hyper = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_maxorder=32, prec_bits=32)
    assert _roundtrip("cpu", SHAPES_CPU, hyper) == 0.0


@pytest.mark.gpu
def test_resume_gpu_4bit(native_lib):
    hyper = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_bits=4)
    assert _roundtrip("cuda:0", SHAPES_GPU, hyper) < 1e-6
