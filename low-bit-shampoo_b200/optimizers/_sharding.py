"""Sharding of the preconditioner work across the GPUs of one node.

The reference is single-device.  Here every parameter that has preconditioner matrices is
owned by one rank (cost-balanced, longest-processing-time-first on a cost model of its
blocks); only the owner holds that parameter's quantized state and runs the statistics
refresh, the inverse root and the preconditioning products.  After the owners have produced
their (norm-grafted) preconditioned gradients, one all-gather over a flat, rank-major fp32
buffer gives every rank every direction, and the AdamW / SGD tail runs replicated.
No other collective is used; gradients are assumed to be already averaged (data parallel).
"""
import torch

from optimizers._base import block_shapes


def param_cost(shape, prec_maxorder):
    """Relative cost of one firing step for a parameter: sum n^3 over its preconditioner orders
    (refresh + inverse root, ~17 n^3 flops each) plus the two apply products per block."""
    cost = 0.0
    for m, k in block_shapes(shape, prec_maxorder):
        cost += 17.0 * (m ** 3 + k ** 3) + 2.0 * (m * m * k + m * k * k)
    return cost


def assign_owners(shapes, world_size, prec_maxorder):
    """Owner rank per parameter (-1 for parameters without preconditioner matrices).

    Deterministic: ties are broken by parameter position, so every rank computes the same map.
    """
    costs = [param_cost(s, prec_maxorder) for s in shapes]
    owners = [-1] * len(shapes)
    load = [0.0] * world_size
    for i in sorted(range(len(shapes)), key=lambda i: (-costs[i], i)):
        if costs[i] == 0.0:
            continue
        r = min(range(world_size), key=lambda r: (load[r], r))
        owners[i] = r
        load[r] += costs[i]
    return owners, load


class GatherPlan:
    """Layout of the flat all-gather buffer: for rank r the directions of the parameters it
    owns, back to back, every rank's slot padded to the largest one."""

    def __init__(self, entries, world_size):
        # entries: list of (key, numel, owner) in a fixed order shared by all ranks
        self.world = world_size
        fill = [0] * world_size
        self.offset = {}
        for key, numel, owner in entries:
            self.offset[key] = (owner, fill[owner], numel)
            fill[owner] += numel
        self.slot = max(1, max(fill))
        self.fill = fill

    def buffers(self, device, dtype):
        """Persistent send / receive buffers (allocated once, so that captured CUDA graphs and the
        eager collective between them always see the same addresses)."""
        buf = getattr(self, "_buffers", None)
        if buf is None or buf[0].device != torch.device(device) or buf[0].dtype != dtype:
            buf = self._buffers = (torch.zeros(self.slot, dtype=dtype, device=device),
                                   torch.empty(self.world * self.slot, dtype=dtype, device=device))
        return buf

    def pack(self, local, rank, device, dtype):
        """Copies this rank's directions ({key: tensor}) into its slot of the send buffer."""
        send, _ = self.buffers(device, dtype)
        keys = list(local)
        if keys:
            dst = []
            for key in keys:
                owner, off, numel = self.offset[key]
                assert owner == rank
                dst.append(send[off: off + numel].view(local[key].shape))
            torch._foreach_copy_(dst, [local[k] for k in keys])

    def collective(self, group, device, dtype):
        """The one exchange step of the sharded optimizer: an all-gather of every rank's slot."""
        import torch.distributed as dist
        send, recv = self.buffers(device, dtype)
        dist.all_gather_into_tensor(recv, send, group=group)

    def views(self, device, dtype):
        """{key: flat view into the receive buffer} for all keys."""
        _, recv = self.buffers(device, dtype)
        recv = recv.view(self.world, self.slot)
        return {key: recv[owner, off: off + numel] for key, (owner, off, numel) in self.offset.items()}

    def exchange(self, local, rank, group, device, dtype):
        """local: {key: tensor} for the keys this rank owns.  Returns {key: flat view} for all keys."""
        self.pack(local, rank, device, dtype)
        self.collective(group, device, dtype)
        return self.views(device, dtype)


def consolidate_state_dicts(shards):
    """Merges the state dicts the ranks of one sharded run saved (optimizer.state_dict() on every
    rank, any order) into one that an optimizer of ANY world size can load: for every parameter
    the entry of the rank that owned it - the only one with real preconditioner state - is kept;
    moments and step counters are replicated, so any rank's copy serves.  The result is tagged
    as a single-process checkpoint; load_state_dict() then re-shards it for the current world."""
    shards = list(shards)
    tags = [sd.get("shampoo_shard") for sd in shards]
    if any(t is None for t in tags):
        raise ValueError("not a Shampoo state dict of this package (no 'shampoo_shard' tag)")
    world = tags[0]["world"]
    if sorted(t["rank"] for t in tags) != list(range(world)) or any(t["world"] != world for t in tags):
        raise ValueError(f"need the state dicts of all {world} ranks of one run, got ranks "
                         f"{sorted(t['rank'] for t in tags)} of worlds {sorted({t['world'] for t in tags})}")
    if any(t["byte_format"] != tags[0]["byte_format"] for t in tags):
        raise ValueError("the shards use different packed-code formats")
    by_rank = {t["rank"]: sd for t, sd in zip(tags, shards)}
    base = by_rank[0]
    state = {}
    for idx, entry in base["state"].items():
        owner = entry.get("owner", -1)
        src = by_rank[owner]["state"][idx] if owner >= 0 else entry
        merged = dict(src)
        merged["owner"] = 0 if owner >= 0 else -1
        state[idx] = merged
    out = {k: v for k, v in base.items() if k not in ("state", "shampoo_shard")}
    out["state"] = state
    out["shampoo_shard"] = {"format": tags[0]["format"], "rank": 0, "world": 1, "byte_format": dict(tags[0]["byte_format"]),
                            "consolidated_from": world}
    return out
