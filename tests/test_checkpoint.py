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


def _resume_variants(device, shapes, hyper, steps=6, cut=3, map_location=None, in_place=False):
    """Like _roundtrip, for options of the restore: `map_location` for torch.load, `in_place`
    loads into the optimizer that wrote the checkpoint (after it has run on) instead of a fresh one."""
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
    ck = torch.load(buf, weights_only=False, map_location=map_location)
    if in_place:
        advance(ps, opt, cut, cut + 2)                      # wander off, then rewind to the checkpoint
        ps2, opt2 = ps, opt
    else:
        ps2, opt2 = make()
    for p, q in zip(ps2, ck["params"]):
        p.data.copy_(q)
    opt2.load_state_dict(ck["opt"])
    advance(ps2, opt2, cut, steps)
    got = [p.detach().cpu() for p in ps2]
    return max(float((a - b).abs().max()) for a, b in zip(got, want)), opt2


@pytest.mark.gpu
@pytest.mark.parametrize("in_place", [False, True])
def test_resume_gpu_4bit_with_cuda_graph(native_lib, in_place):
    """Graph replay after a restore: the captured graphs and pointer tables of the old state are
    dropped, the first step after the load runs eagerly, later ones replay new graphs."""
    hyper = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_bits=4, cuda_graph=True)
    err, opt = _resume_variants("cuda:0", SHAPES_GPU, hyper, steps=8, cut=4, in_place=in_place)
    assert err < 1e-6
    assert opt._use_graph and opt._graph_state is not None and len(opt._graph_state["graphs"]) >= 1


@pytest.mark.gpu
def test_resume_gpu_4bit_from_cpu_mapped_checkpoint(native_lib):
    """torch.load(map_location='cpu') puts the pickled arenas on the host; load_state_dict
    re-creates them on the parameters' device."""
    hyper = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_bits=4)
    err, opt = _resume_variants("cuda:0", SHAPES_GPU, hyper, map_location="cpu")
    assert err < 1e-6
    pre = opt.state[opt.param_groups[0]['params'][0]]['preconditioner']
    cls, slot = pre._slots[0]
    assert cls.stat.var.is_cuda and pre.statistics[0].var.is_cuda
    assert pre.statistics[0].var.data_ptr() == cls.stat.storage(slot)["var"].data_ptr()


def test_state_dict_carries_rank_and_byte_format_tag():
    from optimizers.shampoo2 import ShampooAdamW
    p = torch.nn.Parameter(torch.randn(8, 8))
    opt = ShampooAdamW([p], prec_bits=32)
    p.grad = torch.randn(8, 8)
    opt.step()
    tag = opt.state_dict()["shampoo_shard"]
    assert tag["rank"] == 0 and tag["world"] == 1 and tag["byte_format"]["zero_block_code"] == 0
    bad = opt.state_dict()
    bad["shampoo_shard"] = dict(tag, byte_format=dict(tag["byte_format"], zero_block_code=7))
    with pytest.raises(RuntimeError, match="format"):
        opt.load_state_dict(bad)
    foreign = opt.state_dict()
    foreign["shampoo_shard"] = dict(tag, rank=1, world=2)
    with pytest.raises(RuntimeError, match="rank 1 of 2"):
        opt.load_state_dict(foreign)
