"""GPU parity of the optimizer step with 4-bit state (kernels through the C ABI + batched
engine) against parameters produced by the reference optimizers, and against the CPU oracle.

Tolerance: 1e-4 relative Frobenius error on the post-step parameters."""
import numpy as np
import pytest
import torch

from helpers import load_optimizer_cases, rel_fro
from test_optimizer_host import run_case

pytestmark = pytest.mark.gpu
TOL = 1e-4


def cases(mode):
    _, meta = load_optimizer_cases()
    return [c for c in meta["cases"] if c["mode"] == mode]


@pytest.mark.parametrize("case", cases("bits32"), ids=lambda c: c["key"])
def test_gpu_32bit_step(case, native_lib):
    blob, meta = load_optimizer_cases()
    errs, upd = run_case(blob, meta, case, "cuda:0", 32)
    assert max(errs) < TOL, (errs, upd)


@pytest.mark.parametrize("case", cases("bits4_ret"), ids=lambda c: c["key"])
def test_gpu_4bit_step_vs_reference_with_returning_dequantizer(case, native_lib):
    from optimizers import matrix_functions as MF
    blob, meta = load_optimizer_cases()
    # Schur-Newton cases: the power iteration behind the ridge starts from torch.rand
    # (matrix_functions.py:36).  The fixtures come from the reference on CPU, so the start vectors are
    # drawn from the CPU generator here too, one per matrix in the reference's order.
    MF.START_VECTORS = "host"
    try:
        errs, upd = run_case(blob, meta, case, "cuda:0", 4)
    finally:
        MF.START_VECTORS = "device"
    print(case["key"], "param err", errs, "update err", upd)
    assert max(errs) < TOL, (errs, upd)


@pytest.mark.parametrize("case", cases("bits4"), ids=lambda c: c["key"])
def test_gpu_4bit_step_vs_verbatim_reference(case, native_lib):
    """The unmodified reference: its diagreal dequantizer returns None, so low-bit
    preconditioners act as the identity.  Reproduced with the engine's compatibility flag."""
    from optimizers import _engine
    blob, meta = load_optimizer_cases()
    _engine.REFERENCE_DIAGREAL_NONE = True
    try:
        errs, upd = run_case(blob, meta, case, "cuda:0", 4)
    finally:
        _engine.REFERENCE_DIAGREAL_NONE = False
    print(case["key"], "param err", errs, "update err", upd)
    assert max(errs) < TOL, (errs, upd)


def test_state_objects_are_arena_views(native_lib):
    """Per-parameter QTensor objects alias the batched arenas and decode to the same values."""
    from optimizers.shampoo2 import ShampooAdamW
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(128, 96, device="cuda")), torch.nn.Parameter(torch.randn(96, 128, device="cuda"))]
    opt = ShampooAdamW(ps, prec_bits=4, stat_compute_steps=1, prec_compute_steps=1)
    for p in ps:
        p.grad = torch.randn_like(p)
    opt.step()
    pre = opt.state[ps[0]]["preconditioner"]
    assert len(pre.statistics) == 2 and pre.statistics[0].bits == 4
    cls, slot = pre._slots[0]
    P_obj = pre.preconditioners[0].dequantize()
    P_arena = cls.prec.dequantize(slot, slot + 1)[0]
    assert torch.equal(P_obj, P_arena)
    L_obj, Vt = pre.statistics[0].dequantize()
    assert L_obj.shape == (128, 128) and torch.isfinite(L_obj).all()
    # per-parameter API (reference style) runs on the same state
    out = pre.preconditioned_grad(ps[0].grad)
    assert out.shape == ps[0].shape and torch.isfinite(out).all()


def test_rank_deficient_statistics_stay_finite(native_lib):
    """Non-square blocks give rank-deficient statistics whose small Rayleigh quotients must
    stay accurate relative to the ridge matrix_eps * lambda_max; no NaN may appear."""
    from optimizers.shampoo2 import ShampooAdamW
    torch.manual_seed(3)
    ps = [torch.nn.Parameter(torch.randn(1200, 320, device="cuda") * 0.02),
          torch.nn.Parameter(torch.randn(256, 768, device="cuda") * 0.02)]
    opt = ShampooAdamW(ps, prec_bits=4, stat_compute_steps=1, prec_compute_steps=1)
    for step in range(3):
        for p in ps:
            p.grad = torch.randn_like(p) * 0.01
        opt.step()
        for p in ps:
            assert torch.isfinite(p).all()
    for p in ps:
        pre = opt.state[p]["preconditioner"]
        for q in pre.preconditioners:
            assert torch.isfinite(q.dequantize()).all()
        for s in pre.statistics:
            assert torch.isfinite(s.Svalue).all() and float(s.Svalue.min()) > -1e-6 * float(s.max_eigenvalue)


def test_cuda_graph_step_equals_eager_step(native_lib):
    """Optional graph replay of the whole step: same parameters as the eager step, while the
    parameters' .grad tensors are re-created every step and the schedule alternates phases."""
    from optimizers.shampoo2 import ShampooAdamW
    shapes = [(192, 128), (128,), (96, 320), (64, 64), (1, 1, 48)]
    hyper = dict(lr=1e-2, weight_decay=0.05, prec_bits=4, stat_compute_steps=1, prec_compute_steps=2)

    def run(graph):
        g = torch.Generator().manual_seed(5)
        ps = [torch.nn.Parameter((torch.randn(s, generator=g) * 0.3).cuda()) for s in shapes]
        opt = ShampooAdamW(ps, cuda_graph=graph, **hyper)
        for step in range(6):
            for p in ps:
                p.grad = (torch.randn(p.shape, generator=g) * 0.1).cuda()     # new tensor every step
            opt.step()
        torch.cuda.synchronize()
        return [p.detach().cpu() for p in ps], opt

    eager, _ = run(False)
    graphed, opt = run(True)
    assert opt._graph_state is not None and len(opt._graph_state["graphs"]) >= 2
    for a, b in zip(graphed, eager):
        assert float((a - b).norm() / b.norm()) < 1e-5


def _sharded_worker(rank, world, port, out):
    import os
    import sys
    import torch.distributed as dist
    from conftest import PKG, ROOT
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from optimizers.shampoo2 import ShampooAdamW
        shapes = [(256, 192), (192,), (128, 320), (64, 64), (96, 96)]
        hyper = dict(lr=1e-2, weight_decay=0.05, prec_bits=4, stat_compute_steps=1, prec_compute_steps=1)

        def run(group, graph=False):
            g = torch.Generator().manual_seed(9)
            ps = [torch.nn.Parameter((torch.randn(s, generator=g) * 0.3).cuda()) for s in shapes]
            opt = ShampooAdamW(ps, process_group=group, cuda_graph=graph, **hyper)
            for _ in range(5):
                for p in ps:
                    p.grad = (torch.randn(p.shape, generator=g) * 0.1).cuda()
                opt.step()
            torch.cuda.synchronize()
            assert opt._use_graph == graph                  # a failed capture would have switched it off
            return [p.detach().cpu() for p in ps]

        # eager sharded, sharded with two captured graphs around the eager all-gather, single GPU
        sharded, graphed, single = run(dist.group.WORLD), run(dist.group.WORLD, graph=True), run(None)
        err = max(max(float((a - b).norm() / b.norm()) for a, b in zip(x, single)) for x in (sharded, graphed))
        out.put((rank, err))
    finally:
        dist.destroy_process_group()


def test_sharded_step_on_two_gpus_equals_single_gpu(native_lib):
    """Owner-computes sharding + NCCL all-gather on two GPUs gives the single-GPU parameters.
    (Skipped on a one-GPU machine; the same logic runs on CPU ranks in tests/test_sharding_cpu.py.)"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 1e-5, (rank, err)


def test_fused_adamw_tail_matches_foreach_tail(native_lib):
    """qt_adamw_tail (one multi-tensor launch) against the tensor-wide torch operations of the same
    tail, over several steps with a changing learning rate: parameters and both moments agree to
    fp32 rounding (the fused kernel contracts some multiply-adds)."""
    import copy
    from optimizers import _base
    from optimizers.shampoo2 import ShampooAdamW
    torch.manual_seed(3)
    shapes = [(96, 160), (160,), (64, 96), (7,), (130, 70)]
    ref_params = [torch.randn(s, device="cuda").requires_grad_() for s in shapes]
    new_params = [p.detach().clone().requires_grad_() for p in ref_params]
    kw = dict(lr=1e-2, weight_decay=0.1, prec_bits=4, stat_compute_steps=1, prec_compute_steps=1, start_prec_step=1,
              min_lowbit_size=4096)
    opts = []
    for fused, ps in ((False, ref_params), (True, new_params)):
        _base.FUSED_TAIL = fused
        opts.append(ShampooAdamW(ps, **kw))
    try:
        for step in range(4):
            grads = [torch.randn_like(p) for p in ref_params]
            for fused, opt, ps in ((False, opts[0], ref_params), (True, opts[1], new_params)):
                _base.FUSED_TAIL = fused
                for g in opt.param_groups:
                    g['lr'] = 1e-2 / (step + 1)
                for p, g in zip(ps, grads):
                    p.grad = g.clone()
                opt.step()
    finally:
        _base.FUSED_TAIL = True
    torch.cuda.synchronize()
    assert native_lib.qt_last_error() == 0
    for a, b, oa, ob in zip(ref_params, new_params, opts[0].param_groups[0]['params'], opts[1].param_groups[0]['params']):
        assert float((a.detach() - b.detach()).norm() / a.detach().norm()) < 2e-6
        for k in ('exp_avg', 'exp_avg_sq'):
            x, y = opts[0].state[oa][k], opts[1].state[ob][k]
            assert float((x - y).norm() / x.norm().clamp_min(1e-30)) < 2e-6


def test_adamw_tail_entry_point_handles_unaligned_and_ragged_tensors(native_lib):
    """qt_adamw_tail through the C ABI on tensors that are not 16-byte aligned and whose sizes are
    not multiples of the chunk or of four, against the same arithmetic in torch."""
    import ctypes as ct
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(21)
    sizes = [8192 * 2 + 5, 3, 8192, 4099]
    store = [torch.randn(4, n + 1, device=dev, generator=g) for n in sizes]
    # tensors 0 and 3 start one float into their storage: 4-byte aligned only
    views = [[s[k, (1 if i in (0, 3) else 0):][:n] for k in range(4)] for i, (s, n) in enumerate(zip(store, sizes))]
    for p, d, m, v in views:
        v.abs_()
    beta1, beta2, eps, lr, wd, step = 0.9, 0.999, 1e-8, 1e-2, 0.1, 3
    c0, c1, c2 = 1 / (1 - beta2 ** step) ** 0.5, -lr / (1 - beta1 ** step), 1 - lr * wd
    want = []
    for p, d, m, v in views:
        m2 = m * beta1 + (1 - beta1) * d
        v2 = v * beta2 + (1 - beta2) * d * d
        want.append((p * c2 + c1 * (m2 / (v2.sqrt() * c0 + eps)), m2, v2))
    chunk = 8192
    ct_, ci_ = [], []
    for t, n in enumerate(sizes):
        for c in range((n + chunk - 1) // chunk):
            ct_.append(t)
            ci_.append(c)
    i64 = lambda xs: torch.tensor(xs, dtype=torch.int64, device=dev)
    tabs = [i64([vw[k].data_ptr() for vw in views]) for k in range(4)]
    numels, tct, tci = i64(sizes), torch.tensor(ct_, dtype=torch.int32, device=dev), torch.tensor(ci_, dtype=torch.int32, device=dev)
    scal = torch.tensor([c0, c1, c2], dtype=torch.float32, device=dev)
    vp = lambda t: ct.c_void_p(t.data_ptr())
    rc = native_lib.qt_adamw_tail(vp(tabs[0]), vp(tabs[1]), vp(tabs[2]), vp(tabs[3]), vp(numels), vp(tct), vp(tci), len(ct_), chunk,
                                  vp(scal), beta1, beta2, 1 - beta1, 1 - beta2, eps,
                                  ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    for (p, d, m, v), (wp, wm, wv) in zip(views, want):
        for got, ref in ((p, wp), (m, wm), (v, wv)):
            assert float((got - ref).norm() / ref.norm()) < 1e-6
    # a chunk size that is not a multiple of four is refused, nothing is launched
    assert native_lib.qt_adamw_tail(vp(tabs[0]), vp(tabs[1]), vp(tabs[2]), vp(tabs[3]), vp(numels), vp(tct), vp(tci), len(ct_), 6,
                                    vp(scal), beta1, beta2, 1 - beta1, 1 - beta2, eps, None) != 0


def test_step_with_preconditioners_dequantized_inside_the_products(native_lib):
    """The apply products P_L G P_R with the 4-bit preconditioners dequantized by the product
    kernel's converter warps (every eligible product) give the same parameters as the default
    mix (through operand planes where many output tiles share an operand tile)."""
    from optimizers import _engine
    from optimizers.shampoo2 import ShampooAdamW
    shapes = [(256, 192), (192,), (128, 320), (64, 64), (96, 1216)]
    hyper = dict(lr=1e-2, weight_decay=0.05, prec_bits=4, stat_compute_steps=1, prec_compute_steps=1)

    def run(max_share):
        keep = _engine.DEQUANTIZE_IN_PRODUCT_MAX_SHARE
        _engine.DEQUANTIZE_IN_PRODUCT_MAX_SHARE = max_share
        try:
            g = torch.Generator().manual_seed(13)
            ps = [torch.nn.Parameter((torch.randn(s, generator=g) * 0.3).cuda()) for s in shapes]
            opt = ShampooAdamW(ps, **hyper)
            for _ in range(3):
                for p in ps:
                    p.grad = (torch.randn(p.shape, generator=g) * 0.1).cuda()
                opt.step()
            torch.cuda.synchronize()
            return [p.detach().cpu() for p in ps]
        finally:
            _engine.DEQUANTIZE_IN_PRODUCT_MAX_SHARE = keep

    everywhere, nowhere, mixed = run(None), run(0), run(2)
    assert native_lib.qt_device_error(1) == 0
    for a, b, c in zip(everywhere, nowhere, mixed):
        assert torch.equal(a, b) and torch.equal(c, b)
