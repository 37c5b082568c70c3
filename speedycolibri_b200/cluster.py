"""Expert parallelism: the ownership map of crates/colibri-cluster/src/sharding.rs and the
sharded block of crates/colibri-engine/src/moe.rs:1620-1794, with the reference's TCP
request/response (crates/colibri-cluster/src/net.rs) replaced by NCCL all-to-all over NVLink.

What is kept from the reference: the expert -> rank map (contiguous ``e*N/E`` or an explicit
LPT table), the FNV-1a fingerprint every rank compares before exchanging anything, "move
activations to experts, never weights", and that a peer failure aborts the layer with an
exception rather than returning zeros.  What changes: tokens are sharded across ranks (each
rank routes its own T/world tokens), activations reach the peers through one NCCL all-gather
and the partial sums return through one reduce-scatter, instead of rank 0 driving every peer
with a request/response per layer."""
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


class ShardedMoe:
    """Expert-parallel block over the ranks of `group` (one process per GPU) — the role of
    crates/colibri-engine/src/moe.rs:1737 `moe_sharded`.

    Each rank holds T_local tokens and the experts `sharding` gives it.  Per call, on the current
    stream, with no host synchronisation (every exchanged size follows from T, H, k):

      1. router + top-k of the own tokens                          (block.topk_dev)
      2. all-gather of tokens (overlapped with 1 and 7a), indices, weights   (NCCL)
      3. rows of the (token, kk) pairs routed to resident experts  (block.gather_local_dev)
      4. grouped expert FFN over those rows                        (block.experts_dev)
      5. f32 partial sum per token over the resident experts       (block.combine_partial_dev)
      6. reduce-scatter of the partials: every rank receives the sum for its own tokens (NCCL) —
         the fold of peer partials of moe.rs:1725-1733
      7. + shared expert of the own tokens, one rounding to bf16   (block.shared_dev, finish_dev)

    Like the reference (moe.rs:1671-1678) every rank sees all activation rows and only weights
    never move; unlike it, no rank drives the others.  `block` must be created with
    max_tokens >= world * T_local.  Buffers are allocated once and reused by every call."""

    def __init__(self, block, sharding: ExpertSharding, t_local: int, group=None):
        import torch
        import torch.distributed as dist

        self.block, self.sharding, self.group, self.Tl = block, sharding, group, int(t_local)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world == sharding.num_nodes and self.rank == block.ep_rank
        cfg = block.cfg
        self.k, self.H = cfg.topk, cfg.hidden
        T = self.T = self.world * self.Tl
        assert block.max_tokens >= T, "create the block with max_tokens = tokens of all ranks"
        assert block.local_experts() == sharding.count_for(self.rank)
        self.gloo = dist.get_backend(group) == "gloo"
        dev = "cpu" if self.gloo else torch.device("cuda", block.device)
        bf, i32, f32 = torch.bfloat16, torch.int32, torch.float32
        self.x_all = torch.empty((T, self.H), dtype=bf, device=dev)
        self.idx = torch.empty((self.Tl, self.k), dtype=i32, device=dev)
        self.w = torch.empty((self.Tl, self.k), dtype=f32, device=dev)
        self.idx_all = torch.empty((T, self.k), dtype=i32, device=dev)
        self.w_all = torch.empty((T, self.k), dtype=f32, device=dev)
        self.rows = torch.empty((T * self.k, self.H), dtype=bf, device=dev)
        self.y_rows = torch.empty((T * self.k, self.H), dtype=bf, device=dev)
        self.seg_count = torch.zeros(max(1, block.local_experts()), dtype=i32, device=dev)
        self.slot = torch.empty(T * self.k, dtype=i32, device=dev)
        self.partial = torch.empty((T, self.H), dtype=f32, device=dev)
        self.mine = torch.empty((self.Tl, self.H), dtype=f32, device=dev)
        self.shared_y = torch.empty((self.Tl, self.H), dtype=bf, device=dev) if block.has_shared else None
        self.rows_expected = max(1, T * self.k // self.world)

    def _stream(self):
        import torch

        return 0 if self.gloo else torch.cuda.current_stream().cuda_stream

    STAGES = ("topk", "all_gather", "gather_local", "experts", "combine_partial", "reduce_scatter+shared", "finish")

    def __call__(self, x, out=None, timing=None):
        """`timing`: optional dict that receives per-stage milliseconds (CUDA events on the current
        stream; synchronises at the end, so only for measurement)."""
        import torch
        import torch.distributed as dist

        assert x.shape == (self.Tl, self.H)
        b, st = self.block, self._stream()
        if out is None:
            out = torch.empty_like(x)
        marks = []

        def mark():
            if timing is not None and not self.gloo:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        mark()
        # the token all-gather does not depend on the routing: let it run under the router and the
        # shared expert (NCCL's own stream), and join before the first kernel that reads x_all
        gather_x = None
        if self.gloo:
            dist.all_gather_into_tensor(self.x_all, x, group=self.group)
        else:
            gather_x = dist.all_gather_into_tensor(self.x_all, x, group=self.group, async_op=True)
        b.topk_dev(x, self.idx, self.w, st)
        mark()
        dist.all_gather_into_tensor(self.idx_all, self.idx, group=self.group)
        dist.all_gather_into_tensor(self.w_all, self.w, group=self.group)
        if gather_x is not None:
            gather_x.wait()
        mark()
        b.gather_local_dev(self.x_all, self.idx_all, self.rows, self.seg_count, self.slot, st)
        mark()
        b.experts_dev(self.rows, self.seg_count, self.rows_expected, self.y_rows, st)
        mark()
        b.combine_partial_dev(self.y_rows, self.slot, self.w_all, self.partial, st)
        mark()
        # The shared expert (replicated weights, own tokens) is independent of the exchange: it
        # runs on the compute stream while NCCL reduces the partial sums on its own stream.
        if self.gloo:  # gloo has no reduce-scatter: all-reduce and keep the own slice
            dist.all_reduce(self.partial, group=self.group)
            self.mine.copy_(self.partial[self.rank * self.Tl:(self.rank + 1) * self.Tl])
            if b.has_shared:
                b.shared_dev(x, self.shared_y, st)
        else:
            rs = dist.reduce_scatter_tensor(self.mine, self.partial, group=self.group, async_op=True)
            if b.has_shared:
                b.shared_dev(x, self.shared_y, st)
            rs.wait()
        mark()
        b.finish_dev(self.mine, self.shared_y, out, st)
        mark()
        if marks:
            torch.cuda.synchronize()
            for name, e0, e1 in zip(self.STAGES, marks[:-1], marks[1:]):
                timing[name] = timing.get(name, 0.0) + e0.elapsed_time(e1)
        return out


def moe_sharded(block, sharding: ExpertSharding, x, group=None):
    """One expert-parallel block call; keeps a ShardedMoe (and its buffers) on the block."""
    sm = getattr(block, "_sharded", None)
    if sm is None or sm.Tl != x.shape[0] or sm.sharding is not sharding:
        sm = block._sharded = ShardedMoe(block, sharding, x.shape[0], group)
    return sm(x)
