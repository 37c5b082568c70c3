"""Host logic of expert parallelism on CPU: the sharding maps (crates/colibri-cluster/src/sharding.rs
tests :272-510), the exchange bookkeeping, and a 2-rank gloo run of the counts/rows exchange."""
import os
import subprocess
import sys

import numpy as np
import pytest

from speedycolibri_b200.cluster import ExpertSharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_contiguous_partition():
    sh = ExpertSharding.new(8, 256)
    assert [sh.count_for(n) for n in range(8)] == [32] * 8
    assert sh.owner(0) == 0 and sh.owner(31) == 0 and sh.owner(32) == 1 and sh.owner(255) == 7
    assert sh.range_for(3) == (96, 128)
    sh = ExpertSharding.new(3, 10)  # uneven: within one expert of each other
    counts = [sh.count_for(n) for n in range(3)]
    assert sum(counts) == 10 and max(counts) - min(counts) <= 1
    for n in range(3):
        lo, hi = sh.range_for(n)
        assert sh.local_experts(n) == list(range(lo, hi))
    assert ExpertSharding.single(7).owner_table() == [0] * 7


def test_balanced_is_lpt_and_deterministic():
    w = [100, 1, 1, 1, 50, 50, 1, 1]
    a, b = ExpertSharding.balanced(2, 8, w), ExpertSharding.balanced(2, 8, w)
    assert a.owner_table() == b.owner_table() and a.is_hot_aware()
    assert a.owner(0) != a.owner(4) or a.owner(0) != a.owner(5)  # the hot expert is not stacked with both 50s
    loads = a.node_weights(w)
    assert abs(loads[0] - loads[1]) <= 5
    assert ExpertSharding.balanced(1, 8, w).owner_table() == [0] * 8
    # ties: equal weights -> ids ascending onto nodes ascending
    assert ExpertSharding.balanced(2, 4, [1, 1, 1, 1]).owner_table() == [0, 1, 0, 1]


def test_capacity_weighted_largest_remainder():
    sh = ExpertSharding.capacity_weighted(3, 10, [5, 3, 2], [1] * 10)
    assert [sh.count_for(n) for n in range(3)] == [5, 3, 2]
    sh = ExpertSharding.capacity_weighted(3, 10, [1, 1, 1], [1] * 10)
    assert sorted(sh.count_for(n) for n in range(3)) == [3, 3, 4]
    sh = ExpertSharding.capacity_weighted(2, 6, [0, 0], [3, 2, 1, 1, 1, 1])  # no capacity signal -> balanced
    assert sh.owner_table() == ExpertSharding.balanced(2, 6, [3, 2, 1, 1, 1, 1]).owner_table()
    sh = ExpertSharding.capacity_weighted(2, 4, [1, 0], [1] * 4)  # a node with zero capacity owns nothing
    assert sh.count_for(1) == 0


WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from speedycolibri_b200.cluster import ExpertSharding, ShardedMoe, verify_peers
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), 2
E, k, H, Tl = 8, 2, 16, 6


class Cfg:
    topk, hidden, n_experts = k, H, E


class FakeBlock:
    # Stage calls of MoeBlock restated with torch on the CPU; expert e maps a row x to (e + 1) * x,
    # the shared expert to 0.5 * x.  Only the orchestration in ShardedMoe is under test.
    cfg, device, has_shared = Cfg, 0, True

    def __init__(self, sharding, rank, max_tokens):
        self.ep_rank, self.max_tokens = rank, max_tokens
        self.local = sharding.local_experts(rank)

    def local_experts(self):
        return len(self.local)

    def topk_dev(self, x, idx, w, st):
        v, i = torch.topk(x.float()[:, :E], k, dim=1)
        idx.copy_(i.int())
        w.copy_(torch.softmax(v, dim=1))

    def shared_dev(self, x, y, st):
        y.copy_((x.float() * 0.5).to(y.dtype))

    def gather_local_dev(self, x_all, idx_all, rows, seg_count, slot, st):
        slot.fill_(-1)
        pos = 0
        flat = idx_all.reshape(-1)
        for j, e in enumerate(self.local):
            hit = (flat == e).nonzero().reshape(-1)
            seg_count[j] = len(hit)
            for p in hit.tolist():
                rows[pos] = x_all[p // k]
                slot[p] = pos
                pos += 1

    def experts_dev(self, rows, seg_count, rows_expected, y, st):
        pos = 0
        for j, e in enumerate(self.local):
            n = int(seg_count[j])
            y[pos:pos + n] = (rows[pos:pos + n].float() * (e + 1)).to(y.dtype)
            pos += n

    def combine_partial_dev(self, y_rows, slot, w_all, partial, st):
        partial.zero_()
        for t in range(partial.shape[0]):
            for kk in range(k):
                s = int(slot[t * k + kk])
                if s >= 0:
                    partial[t] += float(w_all[t, kk]) * y_rows[s].float()

    def finish_dev(self, partial, shared_y, out, st):
        out.copy_((partial + shared_y.float()).to(out.dtype))


sh = ExpertSharding.new(world, E)
verify_peers(sh)
blk = FakeBlock(sh, rank, world * Tl)
sm = ShardedMoe(blk, sh, Tl)
g = torch.Generator().manual_seed(5)
x_all = torch.randn((world * Tl, H), generator=g).to(torch.bfloat16)   # same on both ranks
x = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
for rep in range(2):                                                     # buffers are reused
    out = sm(x)
xf = x.float()
v, i = torch.topk(xf[:, :E], k, dim=1)
w = torch.softmax(v, dim=1)
want = torch.zeros_like(xf)
for t in range(Tl):
    for kk in range(k):
        want[t] += w[t, kk] * (xf[t] * (int(i[t, kk]) + 1)).to(torch.bfloat16).float()
want = (want + (xf * 0.5).to(torch.bfloat16).float()).to(torch.bfloat16)
assert torch.allclose(out.float(), want.float(), rtol=2e-2, atol=1e-2), (out.float() - want.float()).abs().max()
# a rank with a different map must be refused before any exchange
try:
    verify_peers(ExpertSharding.balanced(2, E, [rank + 1] + [1] * (E - 1)) if rank == 1 else sh)
    ok = False
except RuntimeError:
    ok = True
flag = torch.tensor([int(ok)]); dist.all_reduce(flag)
assert flag.item() >= 1
dist.destroy_process_group()
print("OK", rank)
"""


def test_two_rank_sharded_block_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = str(29000 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"OK {r}" in o, o
