"""Shared implementation of the two Shampoo flavours.

`shampoo2` keeps each statistic in eigen-factor form (QTensorSVDFast) and `shampoo1`
keeps the dense statistic (QTensorDiagReal); everything else - blocking, schedule,
grafting, the AdamW / SGD tails - is common.  Class and argument names follow the
reference's optimizers/shampoo2.py (BlockPartitioner :35-99, Preconditioner :102-275,
ShampooSGD :278-367, ShampooAdamW :370-468) and optimizers/shampoo1.py.
"""
import ctypes as ct
import itertools
import warnings
import math
from collections import defaultdict

import torch
import torch.optim as optim

import qtensor.functional as F
from qtensor.utils import QTensorDiagReal, QTensorSVDFast
from optimizers import _engine as E

FUSED_TAIL = True              # AdamW tail as one multi-tensor launch of the library (CUDA fp32 parameters)

CODE = 'linear-2'


def cut(d, block_size):
    """Chunk lengths of one dimension of length d: chunks of `block_size` plus a remainder
    (shampoo2.py:50-61); a dimension that fits is left whole."""
    if block_size > 0 and d > block_size:
        full, rest = divmod(d, block_size)
        return [block_size] * full + ([rest] if rest else [])
    return [d]


def matrix_shape(shape):
    """(rows, cols) a parameter is reshaped to (shampoo2.py:115-121), or None when it has fewer
    than two non-unit dimensions (no preconditioner)."""
    dims = [d for d in shape if d != 1]
    if len(dims) < 2:
        return None
    return dims[0], math.prod(dims[1:])


def block_shapes(shape, prec_maxorder):
    """(rows, cols) of the gradient blocks of a parameter, in partition() order.  Pure shape
    arithmetic: the owner map of the sharded optimizer and the optimizer itself both use it."""
    ms = matrix_shape(tuple(shape))
    if ms is None:
        return []
    return list(itertools.product(cut(ms[0], prec_maxorder), cut(ms[1], prec_maxorder)))


class BlockPartitioner:
    """Splits every dimension longer than `block_size` into chunks of `block_size` plus a
    remainder; a tensor becomes the row-major grid of those blocks."""

    def __init__(self, var, block_size):
        self._shape = var.shape
        self._cuts = []                    # per dimension: list of chunk lengths
        self._splits = []                  # (dim, interior cut positions) for split dimensions
        self._split_sizes = []
        for dim, d in enumerate(var.shape):
            sizes = cut(d, block_size)
            self._cuts.append(sizes)
            if len(sizes) > 1:
                self._splits.append((dim, list(itertools.accumulate(sizes))[:-1]))
                self._split_sizes.append((dim, sizes))
        self._num_splits = len(self._cuts)
        self._preconditioner_shapes = []
        for combo in itertools.product(*self._cuts):
            self._preconditioner_shapes.extend([[d, d] for d in combo])

    def shapes_for_preconditioners(self):
        return self._preconditioner_shapes

    def num_splits(self):
        return self._num_splits

    def block_slices(self):
        """Index tuples of the blocks, in partition() order."""
        per_dim = []
        for sizes in self._cuts:
            ends = list(itertools.accumulate(sizes))
            per_dim.append([slice(e - s, e) for s, e in zip(sizes, ends)])
        return list(itertools.product(*per_dim))

    def partition(self, tensor):
        assert tensor.shape == self._shape
        return [tensor[idx] for idx in self.block_slices()]

    def merge_partitions(self, partitions, out=None):
        """The tensor whose blocks are `partitions`; written into `out` (same shape, contiguous) if given."""
        slices = self.block_slices()
        assert len(slices) == len(partitions)
        if len(partitions) == 1:                              # not split: the block is the tensor
            if out is None:
                return partitions[0].reshape(self._shape)
            out.copy_(partitions[0].reshape(self._shape))
            return out
        if len(self._splits) == 1:                            # split along one dimension: one concatenation
            if out is None:
                return torch.cat(list(partitions), dim=self._splits[0][0])
            return torch.cat(list(partitions), dim=self._splits[0][0], out=out)
        if out is None:
            out = torch.empty(self._shape, dtype=partitions[0].dtype, device=partitions[0].device)
        for idx, part in zip(slices, partitions):
            out[idx].copy_(part)
        return out


def _transformed_shape(shape):
    dims = [x for x in shape if x != 1]
    if len(dims) > 1:
        dims = (dims[0], -1)
    return dims


def preconditioner_orders(shape, prec_maxorder):
    """Orders of the preconditioner matrices a parameter of `shape` gets (block-major, axis-minor)."""
    return [n for blk in block_shapes(shape, prec_maxorder) for n in blk]


class Preconditioner:
    """Statistics and inverse-root preconditioners of one parameter."""

    flavour = "s2"

    def __init__(self, var, name2qmap,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64,
                 rect_t1=1, rect_t2=4, inv_root_mode=0, classes=None):
        self.stat_decay = stat_decay
        self.matrix_eps = matrix_eps
        self.inv_root_mode = inv_root_mode
        self._original_shape = var.shape
        self._transformed_shape = _transformed_shape(var.shape)
        reshaped = torch.reshape(var, self._transformed_shape)
        self._partitioner = BlockPartitioner(reshaped, prec_maxorder)
        self._active = False
        self.statistics = []
        self.preconditioners = []
        self._slots = []                                   # (OrderClass, slot) per statistic
        rank = len(self._transformed_shape)
        if rank <= 1:
            return
        if prec_bits in (4, 8) and not var.is_cuda:
            raise RuntimeError("low-bit preconditioner state needs CUDA tensors; this package has no CPU quantizer "
                               "(use prec_bits=32 for CPU runs)")
        device = var.device
        code = name2qmap[CODE].to(device) if prec_bits in (4, 8) else None
        if code is not None:
            name2qmap[CODE] = code
        for shape in self._partitioner.shapes_for_preconditioners():
            n = shape[0]
            if classes is not None:
                cls = classes[n]
            else:
                cls = E.OrderClass(n, 1, device, self.flavour, prec_bits, quan_blocksize, code, min_lowbit_size,
                                   rect_t1, rect_t2)
            slot = cls.alloc()
            self._slots.append((cls, slot))
            common = dict(bits=prec_bits, name2qmap=name2qmap, code=CODE, blocksize=quan_blocksize,
                          min_lowbit_size=min_lowbit_size)
            eye = torch.eye(n, device=device)
            if self.flavour == "s2":
                stat = QTensorSVDFast(matrix_eps * eye, rect_t1=rect_t1, rect_t2=rect_t2, log_prefix=None,
                                      storage=cls.stat_storage(slot), **common)
            else:
                stat = QTensorDiagReal(matrix_eps * eye, storage=cls.stat_storage(slot), **common)
            self.statistics.append(stat)
            self.preconditioners.append(QTensorDiagReal(eye, storage=cls.prec.storage(slot), **common))

    def set_device(self, device):
        """Re-homes the per-matrix holders (reference: shampoo2.py:311-317).  The arenas the batched
        engine works on are re-created on the parameter's device by the optimizer's
        load_state_dict (adopt()), so nothing here has to move them."""
        for s, p in zip(self.statistics, self.preconditioners):
            s.set_device(device)
            p.set_device(device)

    def adopt(self, old):
        """Takes over the schedule flag and the contents of every state slot of `old` (a
        preconditioner restored from a checkpoint, on any device), slot by slot, into this
        object's own arenas."""
        self._active = bool(old.is_active())
        if not self._slots:
            return
        if isinstance(old, RemotePreconditioner) or len(old._slots) != len(self._slots):
            raise RuntimeError(
                f"the checkpoint holds no preconditioner state for a parameter of shape {tuple(self._original_shape)} "
                "that this rank owns: every rank must load the state it saved itself, or a checkpoint merged with "
                "optimizers._sharding.consolidate_state_dicts()")
        for (cn, sn), (co, so) in zip(self._slots, old._slots):
            cn.copy_slot_from(co, sn, so)

    # -- work lists consumed by the batched engine -------------------------------------
    def _grad_blocks(self, grad):
        return self._partitioner.partition(torch.reshape(grad, self._transformed_shape))

    def statistics_items(self, grad):
        rank = len(self._transformed_shape)
        items = []
        for j, g in enumerate(self._grad_blocks(grad)):
            for axis in range(rank):
                cls, slot = self._slots[j * rank + axis]
                items.append((cls, slot, g, axis))
        return items

    def apply_items(self, grad):
        items = []
        for j, g in enumerate(self._grad_blocks(grad)):
            (c0, s0), (c1, s1) = self._slots[2 * j], self._slots[2 * j + 1]
            items.append((c0, s0, c1, s1, g))
        return items

    def merge(self, blocks, out=None):
        """`out`: a contiguous tensor of the parameter's shape that receives the result (or None)."""
        if out is not None:
            out = out.view(self._partitioner._shape)
        return torch.reshape(self._partitioner.merge_partitions(blocks, out), self._original_shape)

    # -- per-parameter entry points (reference API) --------------------------------------
    def _weights(self):
        w1 = self.stat_decay
        return w1, (1.0 if w1 == 1.0 else 1.0 - w1)

    def add_statistics(self, grad):
        if not self.statistics:
            return
        E.add_statistics(self.statistics_items(grad), *self._weights(), eps=self.matrix_eps,
                         exact=(self.inv_root_mode != 0))

    def compute_preconditioners(self):
        if self.statistics:
            E.compute_preconditioners(list(self._slots), self.matrix_eps, self.inv_root_mode)
        self._active = True

    def preconditioned_grad(self, grad):
        if not self.preconditioners:
            return grad
        return self.merge(E.preconditioned_blocks(self.apply_items(grad)))

    def is_active(self) -> bool:
        return self._active


class RemotePreconditioner:
    """Stand-in on the ranks that do not own a parameter's preconditioner state: it follows the
    activation schedule so every rank agrees on when the owner ships a direction."""

    def __init__(self, owner):
        self.owner = owner
        self.statistics = []
        self.preconditioners = []
        self._slots = []
        self._active = False

    def is_active(self):
        return self._active

    def set_device(self, device):
        pass


def _make_codebooks(prec_bits):
    name2qmap = {}
    if prec_bits in (4, 8):
        if CODE == 'dynamic':
            name2qmap[CODE] = F.create_dynamic_map(signed=True, total_bits=prec_bits, power=1)
        elif CODE == 'linear-2':
            name2qmap[CODE] = F.create_linear_map(signed=True, total_bits=prec_bits, power=2)
    return name2qmap


class _ShampooBase(optim.Optimizer):
    """Schedule, state creation and the batched preconditioning pass shared by the SGD and
    AdamW variants.  Subclasses implement `_init_moments` and `_apply_update`."""

    preconditioner_cls = Preconditioner

    def _setup(self, prec_bits, process_group=None):
        self.name2qmap = _make_codebooks(prec_bits)
        self._pg = process_group
        self._world, self._rank = 1, 0
        self._plans = {}
        self._use_graph = False
        self._graph_state = None
        if process_group is not None:
            import torch.distributed as dist
            self._world = dist.get_world_size(process_group)
            self._rank = dist.get_rank(process_group)

    def consumed_params(self):
        """Parameters whose .grad this rank reads in step(): those whose preconditioners it owns and
        those that have none.  The update directions of the others arrive through the exchange, so
        in a sharded run their gradients need not be present on this rank (their .grad may hold
        anything of the right shape).  Before the first step every parameter is listed."""
        out = set()
        for group in self.param_groups:
            for p in group['params']:
                st = self.state.get(p)
                if not st or st.get('owner', -1) in (-1, self._rank):
                    out.add(p)
        return out

    # ---- checkpoint -----------------------------------------------------------------------
    # The reference pickles its Preconditioner objects inside optimizer.state_dict()
    # (train_cifar.py:446-460) and re-homes them in load_state_dict (shampoo2.py:311-317,
    # :403-409).  Same here, plus a tag: which rank of how many wrote the state (a sharded
    # optimizer holds real state only for the parameters it owns) and the byte format of the
    # packed codes (the reference's CPU and CUDA quantizers disagree on nibble order and on the
    # code of an all-zero block; this library writes the CPU quantizer's format).
    BYTE_FORMAT = {"nibble_order": "element 2j in the high nibble of byte j", "zero_block_code": 0,
                   "normalisation": "ieee division", "ties": "lower code"}

    def _check_device_error(self):
        """Raises if one of the library's kernels set the device status word since the last check
        (a bounded wait ran out, or a value left the range of a scaled operand plane: the results
        are then garbage).  Synchronises; called where the caller does anyway."""
        lib = F.lib
        if lib is None:
            return
        devs = {p.device for g in self.param_groups for p in g['params'] if p.device.type == "cuda"}
        for dev in devs:
            with torch.cuda.device(dev):
                rc = lib.qt_device_error(1)
            if rc != 0:
                raise RuntimeError(f"a kernel of libqtensor_b200 reported status {rc} on {dev} "
                                   f"({lib.qt_error_string(rc).decode()}): optimizer state written since the "
                                   "previous check is not valid")

    def state_dict(self):
        self._check_device_error()
        sd = super().state_dict()
        sd["shampoo_shard"] = {"format": 2, "rank": self._rank, "world": self._world,
                               "byte_format": dict(self.BYTE_FORMAT)}
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        shard = state_dict.pop("shampoo_shard", None)
        if shard is not None:
            if shard.get("byte_format", self.BYTE_FORMAT) != self.BYTE_FORMAT:
                raise RuntimeError(f"checkpoint uses another packed-code format: {shard['byte_format']}")
            if shard["world"] != 1 and (shard["world"], shard["rank"]) != (self._world, self._rank):
                raise RuntimeError(
                    f"checkpoint was written by rank {shard['rank']} of {shard['world']}, this is rank {self._rank} of "
                    f"{self._world}: load each rank's own file, or merge the files with "
                    "optimizers._sharding.consolidate_state_dicts() first")
        super().load_state_dict(state_dict)
        # captured graphs, pointer tables and exchange plans refer to the state that was just replaced
        self._graph_state = None
        self._plans = {}
        for name in ("_tail_cache", "_scalar_ring", "_tail_scalars", "_pending_exchange", "_stable_direction_ptrs", "_last_tail_tab"):
            self.__dict__.pop(name, None)
        self._needs_eager = True                           # the next step rebuilds them eagerly
        for group in self.param_groups:
            loaded = [p for p in group['params'] if len(self.state[p]) != 0]
            if loaded:
                self._create_states(group, loaded, adopt=True)
                for p in loaded:
                    self.state[p]['preconditioner'].set_device(p.device)

    def _create_states(self, group, params, adopt=False):
        """One arena per preconditioner order for all new parameters of the group.  With `adopt`
        the parameters already carry state restored from a checkpoint: ownership is recomputed
        for the current world, arenas are created on each parameter's device, and the restored
        slots are copied in (the restored objects themselves are dropped)."""
        new = [p for p in params if adopt or len(self.state[p]) == 0]
        if not new:
            return
        flavour = self.preconditioner_cls.flavour
        owners = [self._rank if preconditioner_orders(p.shape, group['prec_maxorder']) else -1 for p in new]
        if self._world > 1:
            from optimizers._sharding import assign_owners
            owners, _ = assign_owners([tuple(p.shape) for p in new], self._world, group['prec_maxorder'])
        counts = defaultdict(int)
        for p, owner in zip(new, owners):
            if owner not in (-1, self._rank):
                continue
            for n in preconditioner_orders(p.shape, group['prec_maxorder']):
                counts[(p.device, n)] += 1
        bits = group['prec_bits']
        classes = {}
        for (device, n), c in counts.items():
            code = None
            if bits in (4, 8):
                code = self.name2qmap[CODE].to(device)
                self.name2qmap[CODE] = code
            classes.setdefault(device, {})[n] = E.OrderClass(
                n, c, device, flavour, bits, group['quan_blocksize'], code, group['min_lowbit_size'],
                group.get('rect_t1', 1), group.get('rect_t2', 4))
        for p, owner in zip(new, owners):
            state = self.state[p]
            old = state.get('preconditioner') if adopt else None
            if not adopt:
                state['step'] = 0
            state['owner'] = owner
            if owner not in (-1, self._rank):
                state['preconditioner'] = RemotePreconditioner(owner)
                if old is not None:
                    state['preconditioner']._active = bool(old.is_active())
                else:
                    self._init_moments(p, state)
                continue
            pre = self.preconditioner_cls(
                p, self.name2qmap,
                stat_decay=group['stat_decay'], matrix_eps=group['matrix_eps'], prec_maxorder=group['prec_maxorder'],
                prec_bits=bits, min_lowbit_size=group['min_lowbit_size'], quan_blocksize=group['quan_blocksize'],
                rect_t1=group.get('rect_t1', 1), rect_t2=group.get('rect_t2', 4),
                inv_root_mode=group.get('inv_root_mode', 0), classes=classes.get(p.device))
            if old is not None:
                pre.adopt(old)
            else:
                self._init_moments(p, state)
            state['preconditioner'] = pre

    def _tail_direction_views(self, params):
        """Persistent buffers the update directions should be produced in, by parameter index (none here)."""
        return {}

    def _precondition(self, group, params, split_exchange=False):
        """Runs the statistics / inverse-root / apply phases for `params` (all with grads) and
        returns the list of update directions (grafted to the gradient norm where active).
        With `split_exchange` the sharded exchange stops after the pack: the caller then calls
        _exchange_collective() and _exchange_unpack() itself."""
        self._pending_exchange = None
        t1, t2 = group['stat_compute_steps'], group['prec_compute_steps']
        start = group['start_prec_step']
        stat_items, root_items, apply_list = [], [], []
        w1 = group['stat_decay']
        w2 = 1.0 if w1 == 1.0 else 1.0 - w1
        for p in params:
            state = self.state[p]
            state['step'] += 1
            pre = state['preconditioner']
            if state['step'] % t1 == 0 and pre.statistics:
                stat_items += pre.statistics_items(p.grad.data)
        for p in params:
            state = self.state[p]
            pre = state['preconditioner']
            if state['step'] % t2 == 0:
                root_items += pre._slots
                pre._active = True
        if stat_items or root_items:
            E.refresh(stat_items, root_items, w1, w2, group['matrix_eps'], group.get('inv_root_mode', 0),
                      exact=(group.get('inv_root_mode', 0) != 0))
        directions = []
        for p in params:
            state = self.state[p]
            pre = state['preconditioner']
            directions.append(p.grad.data)
            if state['step'] >= start and pre.is_active():
                apply_list.append((len(directions) - 1, p, pre))
        if apply_list:
            items, owner = [], []
            for k, p, pre in apply_list:
                if pre.preconditioners:
                    its = pre.apply_items(p.grad.data)
                    owner.append((k, pre, len(items), len(items) + len(its)))
                    items += its
            blocks = E.preconditioned_blocks(items) if items else []
            # the fused tail reads directions from one persistent buffer: merge straight into it
            tail_views = self._tail_direction_views(params)
            for k, pre, a, b in owner:
                directions[k] = pre.merge(blocks[a:b], out=tail_views.get(k))
            # grafting: rescale the direction to the gradient's norm (shampoo2.py:453).  For
            # parameters without preconditioners the direction IS the gradient, scaled in place.
            ks = [k for k, _, pre in apply_list if not isinstance(pre, RemotePreconditioner)]
            dirs = [directions[k] for k in ks]
            if ks:
                gn = torch._foreach_norm([params[k].grad.data for k in ks])
                dn = torch._foreach_norm(dirs)
                torch._foreach_add_(dn, 1e-12)
                torch._foreach_div_(gn, dn)
                torch._foreach_mul_(dirs, gn)
            if self._world > 1:
                self._pending_exchange = self._exchange_pack(params, directions, apply_list)
        if not split_exchange:
            self._exchange_collective()
            self._exchange_unpack(params, directions)
        return directions

    # The one exchange step of the sharded optimizer, in three parts so that a captured CUDA graph
    # can end after the pack and the next one start at the unpack, with the collective issued
    # eagerly in between (NCCL inside a captured graph did not return on this stack).
    def _exchange_pack(self, params, directions, apply_list):
        from optimizers._sharding import GatherPlan
        shipped = [(k, p) for k, p, pre in apply_list if self.state[p]['owner'] >= 0]
        if not shipped:
            return None
        sig = tuple(k for k, _ in shipped)
        plan = self._plans.get((id(params[0]), sig))
        if plan is None:
            plan = GatherPlan([(k, p.numel(), self.state[p]['owner']) for k, p in shipped], self._world)
            self._plans[(id(params[0]), sig)] = plan
        local = {k: directions[k] for k, p in shipped if self.state[p]['owner'] == self._rank}
        dev = params[shipped[0][0]].device
        plan.pack(local, self._rank, dev, torch.float32)
        return plan, shipped, dev

    def _exchange_collective(self):
        ctx = getattr(self, "_pending_exchange", None)
        if ctx is not None:
            plan, _, dev = ctx
            plan.collective(self._pg, dev, torch.float32)

    def _exchange_unpack(self, params, directions):
        ctx = getattr(self, "_pending_exchange", None)
        self._pending_exchange = None
        if ctx is None:
            return
        plan, shipped, dev = ctx
        got = plan.views(dev, torch.float32)
        stable = set()
        for k, p in shipped:
            if self.state[p]['owner'] != self._rank:
                directions[k] = got[k].view(p.shape).to(p.grad.dtype)
                if directions[k].data_ptr() == got[k].data_ptr():
                    stable.add(got[k].data_ptr())             # lives in the persistent receive buffer
        self._stable_direction_ptrs = stable

    @torch.no_grad()
    def step(self, closure=None):
        self._step_groups()
        self._needs_eager = False

    def _step_groups(self):
        for group in self.param_groups:
            params = [p for p in group['params'] if p.grad is not None]
            for p in params:
                if p.grad.data.is_sparse:
                    raise RuntimeError('Shampoo does not support sparse yet')
            if not params:
                continue
            fresh = any(len(self.state[p]) == 0 for p in params) or self.__dict__.get("_needs_eager", False)
            self._create_states(group, params)
            if self._use_graph and not fresh and self._graph_eligible(group, params):
                self._graph_step(group, params)
            else:
                self._apply_update(group, params)

    # ---- optional CUDA-graph execution of the step --------------------------------------
    def enable_cuda_graph(self, on=True):
        """Replay the whole step (statistics refresh, inverse roots, apply, exchange, AdamW tail)
        as a CUDA graph.  One graph is captured per schedule phase (which intervals fire); the
        first step is always eager (it creates state).  Gradients are copied into buffers owned
        by the optimizer, so parameters' .grad tensors may change address between steps."""
        self._use_graph = bool(on)
        if not on:
            self._graph_state = None

    def _graph_eligible(self, group, params):
        if len(self.param_groups) != 1 or not hasattr(self, "_graph_scalars"):
            return False
        if self.preconditioner_cls.flavour != "s2" or group.get('inv_root_mode', 0) != 0:
            # the Schur-Newton root runs inside the library without host synchronisation when its
            # start vectors are drawn on the device (a capture that meets a host sync falls back to eager)
            from optimizers import matrix_functions as MF
            if MF.START_VECTORS != "device":
                return False
        dev = params[0].device
        if dev.type != "cuda" or any(p.device != dev or p.grad.dtype != torch.float32 for p in params):
            return False
        return len({self.state[p]['step'] for p in params}) == 1

    def _graph_step(self, group, params):
        gs = self._graph_state
        ids = tuple(id(p) for p in params)
        if gs is None or gs["ids"] != ids:
            gs = self._graph_state = {
                "ids": ids, "graphs": {},
                "grads": [torch.empty_like(p.grad) for p in params],
                "scalars": torch.zeros(3, device=params[0].device),
            }
        step = self.state[params[0]]['step'] + 1
        fires_stat = step % group['stat_compute_steps'] == 0
        fires_root = step % group['prec_compute_steps'] == 0
        active = tuple(self.state[p]['preconditioner'].is_active() for p in params)
        key = (fires_stat, fires_root, all(active), any(active), step >= group['start_prec_step'])
        self._stage_scalars(group, step, gs["scalars"])
        # Gradients are staged into the buffers the graphs read.  In a sharded run the gradient of a
        # parameter another rank owns is not read once that parameter is preconditioned (its direction
        # arrives through the exchange), so it is not copied either.
        shipped_now = step >= group['start_prec_step']
        need = [k for k, p in enumerate(params)
                if not (self._world > 1 and shipped_now and self.state[p].get('owner', -1) not in (-1, self._rank)
                        and (fires_root or self.state[p]['preconditioner'].is_active()))]
        torch._foreach_copy_([gs["grads"][k] for k in need], [params[k].grad for k in need])
        user_grads = [p.grad for p in params]
        for p, g in zip(params, gs["grads"]):
            p.grad = g
        try:
            entry = gs["graphs"].get(key)
            if entry is None:
                book = [(self.state[p]['step'], self.state[p]['preconditioner']._active) for p in params]
                lib = F.lib
                before = lib.qt_launch_count() if lib is not None else 0
                graph = torch.cuda.CUDAGraph()
                tail_graph = None
                first_half_ran = False
                try:
                    if self._world == 1:
                        with torch.cuda.graph(graph):
                            self._apply_update(group, params, scalars=gs["scalars"])
                    else:
                        # sharded: graph 1 ends with this rank's directions packed into the send buffer,
                        # the all-gather runs eagerly, graph 2 unpacks and applies the tail
                        with torch.cuda.graph(graph):
                            directions = self._precondition(group, params, split_exchange=True)
                        graph.replay()
                        pending = self._pending_exchange
                        self._exchange_collective()
                        first_half_ran = True
                        tail_graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(tail_graph, pool=graph.pool()):
                            self._exchange_unpack(params, directions)
                            self._apply_tail(group, params, directions, scalars=gs["scalars"])
                except Exception as exc:
                    warnings.warn(f"CUDA-graph capture of the optimizer step failed ({exc!r}); running eagerly")
                    if first_half_ran:                          # statistics, roots and the exchange are done: finish the step
                        self._use_graph = False
                        self._graph_state = None
                        self._pending_exchange = pending
                        self._exchange_unpack(params, directions)
                        self._apply_tail(group, params, directions)
                        return
                    for p, (st, act) in zip(params, book):      # capture failed: undo bookkeeping, go eager
                        self.state[p]['step'] = st
                        self.state[p]['preconditioner']._active = act
                    self._use_graph = False
                    self._graph_state = None
                    self._apply_update(group, params)
                    return
                launches = (lib.qt_launch_count() - before) if lib is not None else 0
                if tail_graph is None:
                    gs["graphs"][key] = (graph, launches, None, None)
                    graph.replay()
                else:
                    gs["graphs"][key] = (graph, launches, tail_graph, pending)
                    tail_graph.replay()                       # graph 1 and the collective already ran above
            else:
                graph, launches, tail_graph, pending = entry
                for p in params:                                # host-side bookkeeping of the captured step
                    st = self.state[p]
                    st['step'] += 1
                    if fires_root:
                        st['preconditioner']._active = True
                graph.replay()
                if tail_graph is not None:
                    self._pending_exchange = pending
                    self._exchange_collective()
                    self._pending_exchange = None
                    tail_graph.replay()
                if F.lib is not None and launches:
                    F.lib.qt_note_graph_replay(launches)
        finally:
            for p, g in zip(params, user_grads):
                p.grad = g


class ShampooSGDBase(_ShampooBase):
    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=0.0, nesterov=False,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64, process_group=None, **extra):
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov,
                        start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                        prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                        prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                        quan_blocksize=quan_blocksize, **extra)
        super().__init__(params, defaults)
        self._setup(prec_bits, process_group)

    def _init_moments(self, p, state):
        state['momentum'] = torch.zeros_like(p, memory_format=torch.preserve_format)

    def _apply_update(self, group, params):
        directions = self._precondition(group, params)
        wd, mom = group['weight_decay'], group['momentum']
        for p, d in zip(params, directions):
            buf = self.state[p]['momentum']
            if wd != 0.0:
                d.add_(p.data, alpha=wd)
            buf.mul_(mom).add_(d)
            upd = d.add(buf, alpha=mom) if group['nesterov'] else buf
            p.data.add_(upd, alpha=-group['lr'])


class ShampooAdamWBase(_ShampooBase):
    def __init__(self, params, lr=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64, process_group=None, cuda_graph=False,
                 **extra):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                        start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                        prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                        prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                        quan_blocksize=quan_blocksize, **extra)
        super().__init__(params, defaults)
        self._setup(prec_bits, process_group)
        self._use_graph = bool(cuda_graph)

    def _init_moments(self, p, state):
        state['exp_avg'] = torch.zeros_like(p, memory_format=torch.preserve_format)
        state['exp_avg_sq'] = torch.zeros_like(p, memory_format=torch.preserve_format)

    def _graph_scalars(self, group, step, out):
        """Step-dependent scalars of the tail, written where a captured graph reads them:
        out[0] = 1 / sqrt(1 - beta2^t), out[1] = -lr / (1 - beta1^t), out[2] = 1 - lr * weight_decay."""
        beta1, beta2 = group['betas']
        out[0] = 1.0 / math.sqrt(1 - beta2 ** step)
        out[1] = -(group['lr'] / (1 - beta1 ** step))
        out[2] = 1 - group['lr'] * group['weight_decay']

    def _stage_scalars(self, group, step, dst):
        """Asynchronous copy of this step's factors to the device through a ring of pinned buffers:
        the host may run several steps ahead of the device, so a buffer is reused only after the
        copy that read it has completed (its event), never by overwriting one still in flight."""
        ring = self.__dict__.setdefault("_scalar_ring", {"next": 0, "slots": []})
        if not ring["slots"]:
            ring["slots"] = [[torch.zeros(3).pin_memory(), None] for _ in range(8)]
        slot = ring["slots"][ring["next"]]
        ring["next"] = (ring["next"] + 1) % len(ring["slots"])
        if slot[1] is not None:
            slot[1].synchronize()
        self._graph_scalars(group, step, slot[0])
        dst.copy_(slot[0], non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record(torch.cuda.current_stream(dst.device))

    # ---- fused tail: one launch of the library's multi-tensor kernel ----------------------
    _TAIL_CHUNK = 8192

    def _fused_tail_ok(self, params, directions):
        if F.lib is None or not FUSED_TAIL or not params:
            return False
        dev = params[0].device
        if dev.type != "cuda" or len({self.state[p]['step'] for p in params}) != 1:
            return False
        for p, d in zip(params, directions):
            st = self.state[p]
            if not (p.device == dev and p.dtype == torch.float32 and p.is_contiguous() and d.dtype == torch.float32
                    and d.is_contiguous() and d.numel() == p.numel() and d.device == dev
                    and st['exp_avg'].is_contiguous() and st['exp_avg_sq'].is_contiguous()
                    and st['exp_avg'].dtype == torch.float32 and st['exp_avg_sq'].dtype == torch.float32):
                return False
        return True

    def _tail_direction_views(self, params):
        """{parameter index: view of the tail's persistent direction buffer} from the table the last
        fused tail used, if it was built for these parameters; empty otherwise (first step, other tail)."""
        last = self.__dict__.get("_last_tail_tab")
        if last is None or not FUSED_TAIL:
            return {}
        key, tab = last
        if len(key) != 2 * len(params) or any(p.data_ptr() != q for p, q in zip(params, key)):
            return {}
        return {k: v for v, k in zip(tab["dviews"], tab["copy_idx"])}

    def _fused_tail(self, group, params, directions, scalars):
        """Decay, both moments and the update for every parameter in one launch (qt_adamw_tail).
        `scalars`: device tensor of the three step-dependent factors."""
        dev = params[0].device
        cache = self.__dict__.setdefault("_tail_cache", {})
        key = tuple(p.data_ptr() for p in params) + tuple(self.state[p]['exp_avg'].data_ptr() for p in params)
        # directions that already sit at a persistent address (views of the exchange's receive buffer)
        # are read where they are; the others are gathered into one persistent buffer
        stable = self.__dict__.get("_stable_direction_ptrs") or ()
        direct = tuple(d.data_ptr() if d.data_ptr() in stable else 0 for d in directions)
        tab = cache.get(("static", key, direct))
        if tab is None and any(direct) and torch.cuda.is_current_stream_capturing():
            # no table for this pattern yet and none can be uploaded while a graph is captured: gather everything
            direct = tuple(0 for _ in directions)
            tab = cache.get(("static", key, direct))
        if tab is None:
            numels = [p.numel() for p in params]
            ct_, ci_ = [], []
            for t, n in enumerate(numels):
                for c in range((n + self._TAIL_CHUNK - 1) // self._TAIL_CHUNK):
                    ct_.append(t)
                    ci_.append(c)
            i64 = lambda xs: torch.tensor(xs, dtype=torch.int64, device=dev)
            # directions are gathered into one persistent buffer (their own tensors move from step to
            # step), so every table is built once - nothing is uploaded while a graph is captured
            copy_idx = [k for k, ptr in enumerate(direct) if not ptr]
            flat = torch.empty(max(4, sum((numels[k] + 3) // 4 * 4 for k in copy_idx)), dtype=torch.float32, device=dev)
            views, dptrs, off = [], list(direct), 0
            for k in copy_idx:
                views.append(flat[off: off + numels[k]].view(params[k].shape))
                dptrs[k] = views[-1].data_ptr()
                off += (numels[k] + 3) // 4 * 4
            tab = cache[("static", key, direct)] = dict(
                p=i64([p.data_ptr() for p in params]), m=i64([self.state[p]['exp_avg'].data_ptr() for p in params]),
                v=i64([self.state[p]['exp_avg_sq'].data_ptr() for p in params]), n=i64(numels),
                d=i64(dptrs), dviews=views, dflat=flat, copy_idx=copy_idx,
                ct=torch.tensor(ct_, dtype=torch.int32, device=dev), ci=torch.tensor(ci_, dtype=torch.int32, device=dev))
        self._last_tail_tab = (key, tab)
        todo = [(v, directions[k]) for v, k in zip(tab["dviews"], tab["copy_idx"]) if directions[k].data_ptr() != v.data_ptr()]
        if todo:                                              # directions that were not produced in place
            torch._foreach_copy_([v for v, _ in todo], [d for _, d in todo])
        beta1, beta2 = group['betas']
        vp = lambda t: ct.c_void_p(t.data_ptr())
        with torch.cuda.device(dev):
            rc = F.lib.qt_adamw_tail(vp(tab["p"]), vp(tab["d"]), vp(tab["m"]), vp(tab["v"]), vp(tab["n"]), vp(tab["ct"]), vp(tab["ci"]),
                                     tab["ct"].numel(), self._TAIL_CHUNK, vp(scalars), float(beta1), float(beta2),
                                     1.0 - float(beta1), 1.0 - float(beta2), float(group['eps']), F._stream(params[0]))
        F._check(rc, "adamw tail")

    def _apply_update(self, group, params, scalars=None):
        directions = self._precondition(group, params)
        self._apply_tail(group, params, directions, scalars)

    def _apply_tail(self, group, params, directions, scalars=None):
        if self._fused_tail_ok(params, directions):
            if scalars is None:                               # eager: stage this step's factors on the device
                scalars = self.__dict__.get("_tail_scalars")
                if scalars is None or scalars.device != params[0].device:
                    scalars = self._tail_scalars = torch.zeros(3, device=params[0].device)
                self._stage_scalars(group, self.state[params[0]]['step'], scalars)
            self._fused_tail(group, params, directions, scalars)
            return
        # decoupled weight decay (shampoo2.py:441; it commutes with the preconditioning, which reads gradients only)
        if scalars is None:
            torch._foreach_mul_(params, 1 - group['lr'] * group['weight_decay'])
        else:
            torch._foreach_mul_(params, scalars[2])
        beta1, beta2 = group['betas']
        by_step = defaultdict(list)
        for k, p in enumerate(params):
            by_step[self.state[p]['step']].append(k)
        for step, ks in by_step.items():
            ps = [params[k] for k in ks]
            ds = [directions[k] for k in ks]
            m1 = [self.state[p]['exp_avg'] for p in ps]
            m2 = [self.state[p]['exp_avg_sq'] for p in ps]
            bc1 = 1 - beta1 ** step
            bc2 = 1 - beta2 ** step
            torch._foreach_mul_(m1, beta1)
            torch._foreach_add_(m1, ds, alpha=1 - beta1)
            torch._foreach_mul_(m2, beta2)
            torch._foreach_addcmul_(m2, ds, ds, value=1 - beta2)
            denom = torch._foreach_sqrt(m2)
            if scalars is None:
                torch._foreach_div_(denom, math.sqrt(bc2))
                torch._foreach_add_(denom, group['eps'])
                torch._foreach_addcdiv_(ps, m1, denom, value=-(group['lr'] / bc1))
            else:                                           # captured graph: scalars live on the device
                torch._foreach_mul_(denom, scalars[0])
                torch._foreach_add_(denom, group['eps'])
                upd = torch._foreach_div(m1, denom)
                torch._foreach_mul_(upd, scalars[1])
                torch._foreach_add_(ps, upd)
