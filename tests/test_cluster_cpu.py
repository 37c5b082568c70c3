"""Host logic of expert parallelism on CPU: the sharding maps (crates/colibri-cluster/src/sharding.rs
tests :272-510), the exchange bookkeeping, and a 2-rank gloo run of the counts/rows exchange."""
import os
import subprocess
import sys

import numpy as np
import pytest

from speedycolibri_b200.cluster import ExpertSharding, exchange_plan

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


def test_exchange_plan_orders_rows_expert_major():
    # 2 ranks, 2 experts each; rank 0's view.  seg_count is in (owner, id) order.
    seg = np.array([3, 1, 2, 4], np.int32)             # my rows to experts 0,1 (mine) and 2,3 (peer)
    recv = np.array([[3, 1], [5, 0]], np.int32)         # rows I receive: from rank 0 and from rank 1
    send, rsplit, perm, per_e = exchange_plan(seg, [2, 2], recv, 0)
    assert send == [4, 6] and rsplit == [4, 5]
    assert per_e.tolist() == [8, 1]
    # received buffer: [r0e0 x3][r0e1 x1][r1e0 x5]; expert-major: e0: r0 rows 0..2 then r1 rows 4..8; e1: row 3
    assert perm.tolist() == [0, 1, 2, 4, 5, 6, 7, 8, 3]


WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from speedycolibri_b200.cluster import ExpertSharding, exchange_plan, verify_peers
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
E, k, H, T = 8, 2, 4, 6
sh = ExpertSharding.new(2, E)
verify_peers(sh)
rng = np.random.default_rng(100 + rank)
idx = np.stack([rng.choice(E, k, replace=False) for _ in range(T)])          # my tokens' experts
order = np.argsort(idx.reshape(-1), kind="stable")                            # (owner,id) order == id order here
rows = torch.tensor((rank * 1000 + order // k)[:, None] * np.ones((1, H)), dtype=torch.float32)  # row payload = token tag
seg = torch.tensor(np.bincount(idx.reshape(-1), minlength=E), dtype=torch.int32)
n_local = [sh.count_for(r) for r in range(2)]
recv_counts = torch.empty(2 * n_local[rank], dtype=torch.int32)
dist.all_to_all_single(recv_counts, seg, output_split_sizes=[n_local[rank]] * 2, input_split_sizes=n_local)
send, rsplit, perm, per_e = exchange_plan(seg.numpy(), n_local, recv_counts.numpy().reshape(2, -1), rank)
recv = torch.empty((sum(rsplit), H))
dist.all_to_all_single(recv, rows, output_split_sizes=rsplit, input_split_sizes=send)
em = recv[torch.from_numpy(perm)]
# every rank checks: rows of my expert j are exactly the tokens (of both ranks) routed to it, source-major
all_idx = [torch.empty((T, k), dtype=torch.int64) for _ in range(2)]
dist.all_gather(all_idx, torch.tensor(idx))
pos = 0
for j, e in enumerate(sh.local_experts(rank)):
    want = [r * 1000 + t for r in range(2) for t in range(T) if e in all_idx[r][t].tolist()]
    got = em[pos:pos + len(want), 0].tolist()
    assert got == want, (rank, e, got, want)
    assert per_e[j] == len(want)
    pos += len(want)
# return trip: y = 2*row back to the source, lands in the sender's original order
y_recv = torch.empty_like(recv); y_recv[torch.from_numpy(perm)] = em * 2
back = torch.empty_like(rows)
dist.all_to_all_single(back, y_recv, output_split_sizes=send, input_split_sizes=rsplit)
assert torch.equal(back, rows * 2)
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


def test_two_rank_exchange_gloo(tmp_path):
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
