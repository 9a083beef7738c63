"""Multi-rank logic on CPU (gloo, world size 2): owner assignment, the all-gather plan and
equality of the sharded optimizer with the single-process one."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def test_owner_assignment_is_balanced_and_deterministic():
    from optimizers._sharding import assign_owners, param_cost
    import workloads
    shapes = [tuple(p.shape) for p in workloads.vit_base_patch32_224().parameters()]
    for world in (2, 4, 8):
        owners, load = assign_owners(shapes, world, 1200)
        again, _ = assign_owners(shapes, world, 1200)
        assert owners == again
        assert max(load) / (sum(load) / world) < 1.05
        for s, o in zip(shapes, owners):
            assert (o == -1) == (param_cost(s, 1200) == 0.0)
            assert -1 <= o < world
    # vectors and scalars-with-unit-dims never get an owner
    assert assign_owners([(768,), (1, 1, 768), (10, 1)], 4, 1200)[0] == [-1, -1, -1]


def test_gather_plan_layout():
    from optimizers._sharding import GatherPlan
    plan = GatherPlan([("a", 10, 0), ("b", 4, 1), ("c", 6, 0), ("d", 1, 1)], 2)
    assert plan.slot == 16 and plan.fill == [16, 5]
    assert plan.offset["c"] == (0, 10, 6) and plan.offset["d"] == (1, 4, 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, flavour, out):
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from optimizers import shampoo1, shampoo2
        mod = shampoo2 if flavour == "s2" else shampoo1
        shapes = [(40, 24), (24,), (24, 40), (8, 3, 3, 3), (1, 1, 16), (56, 56), (20, 64)]
        hyper = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_maxorder=32,
                     prec_bits=32)

        def run(group):
            g = torch.Generator().manual_seed(7)
            ps = [torch.nn.Parameter(torch.randn(s, generator=g)) for s in shapes]
            opt = mod.ShampooAdamW(ps, process_group=group, **hyper)
            for step in range(4):
                for p in ps:
                    p.grad = torch.randn(p.shape, generator=g) * 0.1
                torch.manual_seed(step)
                opt.step()
            return ps, opt

        sharded, opt = run(dist.group.WORLD)
        single, _ = run(None)
        err = max(float((a.detach() - b.detach()).abs().max()) for a, b in zip(sharded, single))
        owned = sum(1 for p in sharded if opt.state[p]["owner"] == rank)
        remote = sum(1 for p in sharded if opt.state[p]["owner"] not in (-1, rank))
        states = sum(len(opt.state[p]["preconditioner"].statistics) for p in sharded)
        out.put((rank, err, owned, remote, states))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("flavour", ["s2", "s1"])
def test_sharded_step_equals_single_process(flavour):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, flavour, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    total_states = 0
    for rank, err, owned, remote, states in results:
        # the dense flavour draws its power-iteration start per batch, and a rank's batches hold
        # fewer matrices than the single process's, so the ridge estimate differs slightly
        assert err < (1e-6 if flavour == "s2" else 1e-4), (rank, err)
        assert owned > 0 and remote > 0          # work and state are really split
        total_states += states
    assert total_states == 4 + 4 + 2 + 8 + 4         # every matrix has exactly one owner


SHAPES_CK = [(40, 24), (24,), (24, 40), (8, 3, 3, 3), (56, 56), (20, 64)]
HYPER_CK = dict(lr=1e-2, weight_decay=0.05, stat_compute_steps=1, prec_compute_steps=2, prec_maxorder=32, prec_bits=32)


def _ck_grads(steps):
    g = torch.Generator().manual_seed(11)
    return [[torch.randn(s, generator=g) * 0.1 for s in SHAPES_CK] for _ in range(steps)]


def _ck_make(group):
    from optimizers.shampoo2 import ShampooAdamW
    g = torch.Generator().manual_seed(7)
    ps = [torch.nn.Parameter(torch.randn(s, generator=g)) for s in SHAPES_CK]
    return ps, ShampooAdamW(ps, process_group=group, **HYPER_CK)


def _ck_advance(ps, opt, grads, lo, hi):
    for t in range(lo, hi):
        for p, gr in zip(ps, grads[t]):
            p.grad = gr.clone()
        opt.step()


def _ck_worker(rank, world, port, folder, out):
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        grads = _ck_grads(6)
        ps, opt = _ck_make(dist.group.WORLD)
        _ck_advance(ps, opt, grads, 0, 3)
        torch.save({"opt": opt.state_dict(), "params": [p.detach().clone() for p in ps]},
                   os.path.join(folder, f"rank{rank}.pt"))
        _ck_advance(ps, opt, grads, 3, 6)
        want = [p.detach().clone() for p in ps]
        dist.barrier()
        # every rank reloads its own file into a fresh sharded optimizer and continues
        ck = torch.load(os.path.join(folder, f"rank{rank}.pt"), weights_only=False)
        ps2, opt2 = _ck_make(dist.group.WORLD)
        for p, q in zip(ps2, ck["params"]):
            p.data.copy_(q)
        opt2.load_state_dict(ck["opt"])
        _ck_advance(ps2, opt2, grads, 3, 6)
        err = max(float((a.detach() - b).abs().max()) for a, b in zip(ps2, want))
        # another rank's file is refused instead of silently dropping the preconditioning
        other = torch.load(os.path.join(folder, f"rank{1 - rank}.pt"), weights_only=False)
        refused = False
        try:
            _ck_make(dist.group.WORLD)[1].load_state_dict(other["opt"])
        except RuntimeError:
            refused = True
        if rank == 0:
            torch.save(want, os.path.join(folder, "want.pt"))
        out.put((rank, err, refused))
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_reloads_per_rank_and_onto_another_world_size(tmp_path):
    """Rank-tagged state dicts of a two-rank run: (i) each rank resumes from its own file;
    (ii) a foreign file is refused; (iii) the two files merged by consolidate_state_dicts()
    resume in a single process (world size 1) to the same parameters."""
    from optimizers._sharding import consolidate_state_dicts
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ck_worker, args=(r, 2, port, str(tmp_path), out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, refused in results:
        assert err < 1e-6 and refused, (rank, err, refused)
    files = [torch.load(tmp_path / f"rank{r}.pt", weights_only=False) for r in range(2)]
    assert [f["opt"]["shampoo_shard"]["rank"] for f in files] == [0, 1]
    with pytest.raises(ValueError):
        consolidate_state_dicts([files[0]["opt"]])           # a rank is missing
    merged = consolidate_state_dicts([f["opt"] for f in reversed(files)])
    assert merged["shampoo_shard"]["world"] == 1
    want = torch.load(tmp_path / "want.pt", weights_only=False)
    grads = _ck_grads(6)
    ps, opt = _ck_make(None)
    for p, q in zip(ps, files[0]["params"]):
        p.data.copy_(q)
    opt.load_state_dict(merged)
    for p in ps:
        assert len(opt.state[p]["preconditioner"].statistics) == (0 if p.dim() < 2 else len(opt.state[p]["preconditioner"]._slots))
    _ck_advance(ps, opt, grads, 3, 6)
    err = max(float((a.detach() - b).abs().max()) for a, b in zip(ps, want))
    assert err < 1e-6, err
