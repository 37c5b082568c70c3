"""Expert parallelism: the ownership map of crates/colibri-cluster/src/sharding.rs and the
sharded block of crates/colibri-engine/src/moe.rs:1620-1794, with the reference's TCP
request/response (crates/colibri-cluster/src/net.rs) replaced by NCCL all-to-all over NVLink.

What is kept from the reference: the expert -> rank map (contiguous ``e*N/E`` or an explicit
LPT table), the FNV-1a fingerprint every rank compares before exchanging anything, "move
activations to experts, never weights", and that a peer failure aborts the layer with an
exception rather than returning zeros.  What changes: tokens are sharded across ranks (each
rank routes its own T/world tokens) and only the rows a peer's experts need are sent, instead
of rank 0 broadcasting every activation row to every peer."""
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


def exchange_plan(seg_count: np.ndarray, n_local: Sequence[int], recv_counts: np.ndarray, rank: int):
    """Host-side bookkeeping of the dispatch all-to-all.

    seg_count  [E]            rows this rank routes to each expert, in (owner, id) order
    n_local    [world]        experts owned by each rank
    recv_counts [world, n_local[rank]]  rows each source rank sends for each of my experts
    Returns (send_splits, recv_splits, perm, rows_per_local_expert): `perm` reorders the
    received rows from [source][expert] order into expert-major order (all sources' rows of
    my first expert, then of my second, ...), sources ascending inside an expert — the order
    in which the reference folds peer partials (moe.rs:1725-1733)."""
    world = len(n_local)
    bounds = np.concatenate([[0], np.cumsum(n_local)])
    send_splits = [int(seg_count[bounds[r]:bounds[r + 1]].sum()) for r in range(world)]
    recv_splits = [int(recv_counts[r].sum()) for r in range(world)]
    nl = int(n_local[rank])
    c = recv_counts.reshape(world, nl).astype(np.int64)
    src_off = np.concatenate([[0], np.cumsum(c.reshape(-1))])[:-1].reshape(world, nl)
    total = int(c.sum())
    perm = np.empty(total, np.int64)
    pos = 0
    for e in range(nl):
        for s in range(world):
            n = int(c[s, e])
            perm[pos:pos + n] = src_off[s, e] + np.arange(n)
            pos += n
    return send_splits, recv_splits, perm, c.sum(axis=0).astype(np.int32)


def moe_sharded(block, sharding: ExpertSharding, x, group=None):
    """Expert-parallel block over the ranks of `group` (one process per GPU).

    `x` is this rank's token shard, torch bf16 CUDA [T_local, H]; returns this rank's
    [T_local, H].  Steps: route + permute locally -> counts all-to-all -> rows all-to-all ->
    local experts (grouped FFN) -> rows all-to-all back -> weighted combine + shared expert
    at the home rank.  The two row exchanges are ncclSend/ncclRecv groups issued through
    torch.distributed.all_to_all_single on the current stream."""
    import torch
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    assert world == sharding.num_nodes and rank == block.ep_rank
    cfg = block.cfg
    E, k, H = cfg.n_experts, cfg.topk, cfg.hidden
    T = x.shape[0]
    dev = x.device
    st = torch.cuda.current_stream(dev).cuda_stream
    n_local = [sharding.count_for(r) for r in range(world)]
    first_seg = sum(n_local[:rank])
    nl = n_local[rank]

    rows = torch.empty((T * k, H), dtype=torch.bfloat16, device=dev)
    seg_count = torch.empty(E, dtype=torch.int32, device=dev)
    slot = torch.empty(max(T * k, 1), dtype=torch.int32, device=dev)
    block.route_dev(x, rows, seg_count, slot, st)

    shared_y = None
    if block.has_shared:  # replicated weights, own tokens; independent of the exchange
        shared_y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        block.shared_dev(x, shared_y, st)

    recv_counts = torch.empty(world * nl, dtype=torch.int32, device=dev)
    dist.all_to_all_single(recv_counts, seg_count, output_split_sizes=[nl] * world, input_split_sizes=n_local, group=group)
    seg_h = seg_count.cpu().numpy()
    rc_h = recv_counts.cpu().numpy().reshape(world, nl)
    send_splits, recv_splits, perm_h, per_expert = exchange_plan(seg_h, n_local, rc_h, rank)
    n_recv = int(sum(recv_splits))

    recv = torch.empty((n_recv, H), dtype=torch.bfloat16, device=dev)
    dist.all_to_all_single(recv, rows, output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)

    perm = torch.from_numpy(perm_h).to(dev, non_blocking=True)
    rows_em = recv.index_select(0, perm) if n_recv else recv
    y_em = torch.empty_like(rows_em)
    cnt_dev = torch.from_numpy(per_expert).to(dev, non_blocking=True)
    block.experts_dev(rows_em, cnt_dev, first_seg, nl, n_recv, y_em, st)
    y_recv = torch.empty_like(recv)
    if n_recv:
        y_recv.index_copy_(0, perm, y_em)

    y_rows = torch.empty_like(rows)
    dist.all_to_all_single(y_rows, y_recv, output_split_sizes=send_splits, input_split_sizes=recv_splits, group=group)

    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    block.combine_dev(y_rows, slot, shared_y, out, st)
    return out
