"""Expert parallelism: the ownership map of crates/colibri-cluster/src/sharding.rs and the
sharded block of crates/colibri-engine/src/moe.rs:1620-1794, with the reference's TCP
request/response (crates/colibri-cluster/src/net.rs) replaced by an all-to-all of token rows inside
one library call: rows stored straight into the peers' receive buffers over NVLink (default), or
exchanged with NCCL send/recv.

What is kept from the reference: the expert -> rank map (contiguous ``e*N/E`` or an explicit
LPT table), the FNV-1a fingerprint every rank compares before exchanging anything, "move
activations to experts, never weights", and that a peer failure aborts the layer with an
exception rather than returning zeros.  What changes: tokens are sharded across ranks (each
rank routes its own tokens), a token row visits each rank that owns one of its experts once,
and the unweighted expert outputs come back to the token's home rank, which combines them —
instead of rank 0 driving every peer with all of x and folding [T,H] partial sums."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np


class ExpertSharding:
    """crates/colibri-cluster/src/sharding.rs:56-266."""

    def __init__(self, num_nodes: int, n_experts: int, table: Optional[Sequence[int]] = None):
        assert num_nodes >= 1, "num_nodes must be >= 1"
        assert n_experts >= 1, "n_experts must be >= 1"
        self.num_nodes, self.n_experts = int(num_nodes), int(n_experts)
        self.table = None if table is None else [int(v) for v in table]

    # sharding.rs:69-78
    @classmethod
    def new(cls, num_nodes: int, n_experts: int) -> "ExpertSharding":
        return cls(num_nodes, n_experts)

    @classmethod
    def single(cls, n_experts: int) -> "ExpertSharding":
        return cls(1, n_experts)

    # sharding.rs:87-109 — LPT greedy, heaviest expert first onto the lightest node, ties by id
    @classmethod
    def balanced(cls, num_nodes: int, n_experts: int, weights: Sequence[int]) -> "ExpertSharding":
        if num_nodes == 1:
            return cls.single(n_experts)
        w = lambda e: int(weights[e]) if e < len(weights) else 0
        order = sorted(range(n_experts), key=lambda e: (-w(e), e))
        load = [0] * num_nodes
        table = [0] * n_experts
        for e in order:
            node = min(range(num_nodes), key=lambda i: (load[i], i))
            table[e] = node
            load[node] += w(e)
        return cls(num_nodes, n_experts, table)

    # sharding.rs:131-189 — largest-remainder quotas by capacity, then LPT under quota
    @classmethod
    def capacity_weighted(cls, num_nodes: int, n_experts: int, capacity: Sequence[int], weights: Sequence[int]):
        cap = lambda n: int(capacity[n]) if n < len(capacity) else 0
        total = sum(cap(n) for n in range(num_nodes))
        if num_nodes == 1 or total == 0:
            return cls.balanced(num_nodes, n_experts, weights)
        quota, rem, assigned = [0] * num_nodes, [], 0
        for n in range(num_nodes):
            exact = cap(n) * n_experts
            quota[n] = exact // total
            assigned += quota[n]
            rem.append((exact % total, n))
        rem.sort(key=lambda r: (-r[0], r[1]))
        for _, n in rem[: n_experts - assigned]:
            quota[n] += 1
        w = lambda e: int(weights[e]) if e < len(weights) else 0
        order = sorted(range(n_experts), key=lambda e: (-w(e), e))
        load, used, table = [0] * num_nodes, [0] * num_nodes, [0] * n_experts
        for e in order:
            node = min((i for i in range(num_nodes) if used[i] < quota[i]), key=lambda i: (load[i], i))
            table[e] = node
            used[node] += 1
            load[node] += w(e)
        return cls(num_nodes, n_experts, table)

    def is_hot_aware(self) -> bool:
        return self.table is not None

    # sharding.rs:197-203
    def owner(self, expert: int) -> int:
        assert 0 <= expert < self.n_experts
        if self.table is not None:
            return self.table[expert]
        return expert * self.num_nodes // self.n_experts

    def is_local(self, node: int, expert: int) -> bool:
        return self.owner(expert) == node

    # sharding.rs:215-224 (contiguous maps only)
    def range_for(self, node: int):
        assert self.table is None, "range_for is contiguous-only"
        e, n = self.n_experts, self.num_nodes
        return (-(-node * e // n), -(-(node + 1) * e // n))

    def count_for(self, node: int) -> int:
        return sum(1 for e in range(self.n_experts) if self.owner(e) == node)

    def local_experts(self, node: int) -> List[int]:
        return [e for e in range(self.n_experts) if self.owner(e) == node]

    def node_weights(self, weights: Sequence[int]) -> List[int]:
        out = [0] * self.num_nodes
        for e in range(self.n_experts):
            out[self.owner(e)] += int(weights[e]) if e < len(weights) else 0
        return out

    def owner_table(self) -> List[int]:
        return [self.owner(e) for e in range(self.n_experts)]

    # sharding.rs:251-265
    def fingerprint(self) -> int:
        h = 0xCBF29CE484222325
        def mix(x):
            nonlocal h
            for b in int(x).to_bytes(4, "little"):
                h ^= b
                h = (h * 0x00000100000001B3) & 0xFFFFFFFFFFFFFFFF
        mix(self.num_nodes)
        mix(self.n_experts)
        for e in range(self.n_experts):
            mix(self.owner(e))
        return h


def verify_peers(sharding: ExpertSharding, group=None) -> None:
    """Every rank must hold the identical map before the first exchange — the handshake of
    crates/colibri-cluster/src/net.rs:324-364,445-458.  Raises on a mismatch."""
    import torch
    import torch.distributed as dist

    fp = sharding.fingerprint()
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.tensor([fp & 0x7FFFFFFF, fp >> 31 & 0x7FFFFFFF, fp >> 62], dtype=torch.int64, device=dev)
    allv = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(allv, mine, group=group)
    for r, v in enumerate(allv):
        if not torch.equal(v.cpu(), mine.cpu()):
            raise RuntimeError(f"sharding fingerprint mismatch: rank {r} disagrees with rank {dist.get_rank(group)} ({fp:#018x})")


def ep_layout(table: np.ndarray, rank: int) -> dict:
    """The segment layout rank `rank` derives from the count table [world, 2, world] of an
    expert-parallel call (``coli_b200_ep_layout``, host-only)."""
    from . import _lib
    from .backend import _check

    table = np.ascontiguousarray(table, dtype=np.int32)
    world = table.shape[0]
    out = np.zeros((8, world), np.int32)
    _check(_lib.load().coli_b200_ep_layout(table.ctypes.data, world, rank, out.ctypes.data), "coli_b200_ep_layout")
    names = ("send_tok", "send_pair", "recv_tok", "recv_pair", "send_off", "recv_off", "ret_send_off", "ret_recv_off")
    return {n: out[i].copy() for i, n in enumerate(names)}


def rows_per_rank(table: np.ndarray) -> np.ndarray:
    """Expert rows (token, kk pairs) each rank computes in a call with this count table."""
    return np.asarray(table)[:, 1, :].sum(axis=0)


def ep_communicator(device: int, group=None) -> int:
    """An ncclComm_t (as an integer) over the ranks of `group`, made by the library itself: rank 0
    draws the 128-byte id, torch.distributed carries it to the others (any backend), every rank
    joins.  The caller destroys it with ``destroy_communicator`` after the handles that use it."""
    import ctypes as C

    import torch.distributed as dist

    from . import _lib
    from .backend import _check

    lib = _lib.load()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [None]
    if rank == 0:
        buf = (C.c_char * 128)()
        _check(lib.coli_b200_nccl_unique_id(buf), "coli_b200_nccl_unique_id")
        box[0] = bytes(buf)
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    comm = C.c_void_p()
    _check(lib.coli_b200_nccl_comm_create(C.byref(comm), box[0], rank, world, device), "coli_b200_nccl_comm_create")
    return comm.value


def destroy_communicator(comm: int) -> None:
    from . import _lib

    if comm:
        _lib.load().coli_b200_nccl_comm_destroy(comm)


class ShardedMoe:
    """Expert-parallel block over the ranks of `group` (one process per GPU) — the role of
    crates/colibri-engine/src/moe.rs:1737 `moe_sharded`.  A thin owner of the pieces: the sharding
    (verified against the peers), the communicator and the ``MoeBlock`` handle created with both;
    a call is ONE library call per rank (``coli_b200_moe_block_ep_dev``).

    `layer` holds the experts ``sharding`` gives this rank (others None) and the shared expert;
    `max_tokens` bounds the tokens of ALL ranks in one call."""

    def __init__(self, cfg, layer, sharding: ExpertSharding, max_tokens: int, device: int, group=None):
        import torch.distributed as dist

        from .moe import MoeBlock

        self.sharding, self.group = sharding, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world == sharding.num_nodes
        verify_peers(sharding, group)
        self.comm = ep_communicator(device, group)
        self.block = MoeBlock(cfg, layer, max_tokens, device=device, ep_rank=self.rank, ep_world=self.world,
                              expert_owner=sharding.owner_table() if sharding.is_hot_aware() else None, nccl_comm=self.comm)
        assert self.block.local_experts() == sharding.count_for(self.rank)

    def __call__(self, x, out=None):
        return self.block.forward_ep(x, out)

    def stage_ms(self, x, steps: int):
        """Per-stage milliseconds, the median over `steps` extra calls (every rank must take part).

        The stages that end in a barrier also hold the time this rank waited for the slowest peer to
        reach it, so one stalled host anywhere in the job shows up in every rank's figure for that
        call; the median keeps a single such call from setting the figure."""
        import numpy as np

        self.block.ep_profile(True)
        per_call, prev = [], None
        for _ in range(steps):
            self.block.forward_ep(x)
            ms, calls = self.block.ep_stage_ms()  # cumulative since profiling was switched on
            cur = dict(ms)
            per_call.append({k: cur[k] - (prev[k] if prev else 0.0) for k in cur})
            prev = cur
        self.block.ep_profile(False)
        return {k: float(np.median([c[k] for c in per_call])) for k in per_call[0]} if per_call else {}

    def close(self):
        import torch

        torch.cuda.synchronize()
        self.block.close()
        destroy_communicator(self.comm)
        self.comm = None
