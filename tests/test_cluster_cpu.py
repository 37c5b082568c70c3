"""Host logic of expert parallelism on CPU: the sharding maps (crates/colibri-cluster/src/sharding.rs
tests :272-510), the exchange layout, and 2- and 3-rank gloo runs of the counts/rows exchange."""
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
# Two gloo ranks on CPU carry out the expert-parallel exchange exactly as the library lays it out:
# each rank plans its dispatch (stated here in numpy: a token goes once to every rank that owns one
# of its experts, tokens ascending), the counts are all-gathered, BOTH sides derive their segment
# offsets from the table with the library's own host function, rows travel with send/recv, a toy
# expert (row * (e + 1)) runs on the owner, results return in (source, token, kk) order and the home
# rank combines.  What is under test is that sender and receiver agree on every offset.
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from speedycolibri_b200.cluster import ExpertSharding, ep_layout, verify_peers
world = int(sys.argv[4])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=world)
rank = dist.get_rank()
E, k, H = 12, 3, 8
Tl = [7, 4, 5][rank]                       # ragged token counts
sh = ExpertSharding.balanced(world, E, [5, 1, 1, 9, 1, 1, 2, 2, 7, 1, 1, 3])
verify_peers(sh)
own = np.array(sh.owner_table())
rng = np.random.default_rng(100 + rank)
x = rng.standard_normal((Tl, H)).astype(np.float32)
idx = np.stack([rng.choice(E, k, replace=False) for _ in range(Tl)]).astype(np.int32)
w = rng.random((Tl, k)).astype(np.float32)
peer_order = lambda r: [r] + [p for p in range(world) if p != r]
# plan (device kernel k_ep_plan, restated)
tok_list = {d: [t for t in range(Tl) if (own[idx[t]] == d).any()] for d in range(world)}
pairs = {d: [(t, kk) for t in range(Tl) for kk in range(k) if own[idx[t, kk]] == d] for d in range(world)}
cnt = torch.tensor([len(tok_list[d]) for d in range(world)] + [len(pairs[d]) for d in range(world)], dtype=torch.int32)
allc = [torch.empty_like(cnt) for _ in range(world)]
dist.all_gather(allc, cnt)
table = torch.stack(allc).numpy().reshape(world, 2, world)
lay = ep_layout(table, rank)
assert list(lay["send_tok"]) == [len(tok_list[d]) for d in range(world)]
R = int(lay["recv_tok"].sum())
recv_x = torch.zeros((max(R, 1), H)); recv_idx = torch.zeros((max(R, 1), k), dtype=torch.int32)
send_rows = int(sum(lay["send_tok"][p] for p in range(world) if p != rank))
send_x = torch.zeros((max(send_rows, 1), H)); send_idx = torch.zeros((max(send_rows, 1), k), dtype=torch.int32)
for d in range(world):                      # pack (k_ep_pack): own rows straight into the receive buffer
    for j, t in enumerate(tok_list[d]):
        if d == rank:
            recv_x[j] = torch.from_numpy(x[t]); recv_idx[j] = torch.from_numpy(idx[t])
        else:
            send_x[lay["send_off"][d] + j] = torch.from_numpy(x[t]); send_idx[lay["send_off"][d] + j] = torch.from_numpy(idx[t])
def exchange(bufs):                         # bufs: list of (send tensor slice or None, recv tensor slice or None, peer)
    reqs = []
    for snd, rcv, p in bufs:
        if rcv is not None: reqs.append(dist.irecv(rcv, src=p))
    for snd, rcv, p in bufs:
        if snd is not None: reqs.append(dist.isend(snd.contiguous(), dst=p))
    for r in reqs: r.wait()
seg = lambda buf, off, n: buf[off:off + n] if n > 0 else None
peers = [p for p in range(world) if p != rank]
exchange([(seg(send_x, lay["send_off"][p], lay["send_tok"][p]), seg(recv_x, lay["recv_off"][p], lay["recv_tok"][p]), p) for p in peers])
exchange([(seg(send_idx, lay["send_off"][p], lay["send_tok"][p]), seg(recv_idx, lay["recv_off"][p], lay["recv_tok"][p]), p) for p in peers])
# owner side: every received pair that hits a resident expert, in (segment, token, kk) order
stream = [recv_x[j] * float(int(recv_idx[j, kk]) + 1) for j in range(R) for kk in range(k) if own[int(recv_idx[j, kk])] == rank]
assert len(stream) == int(lay["recv_pair"].sum())
self_pairs = int(lay["recv_pair"][rank])
ret_recv = torch.zeros((max(int(lay["send_pair"].sum()), 1), H))
for j in range(self_pairs): ret_recv[j] = stream[j]
ret_send = torch.stack(stream[self_pairs:]) if len(stream) > self_pairs else torch.zeros((1, H))
exchange([(seg(ret_send, lay["ret_send_off"][p], lay["recv_pair"][p]), seg(ret_recv, lay["ret_recv_off"][p], lay["send_pair"][p]), p) for p in peers])
# home side: pair (t, kk) owned by d sits at ret_recv_off[d] + its rank among d's pairs
out = np.zeros((Tl, H), np.float32)
for d in range(world):
    for j, (t, kk) in enumerate(pairs[d]):
        out[t] += w[t, kk] * ret_recv[lay["ret_recv_off"][d] + j].numpy()
want = np.zeros((Tl, H), np.float32)
for t in range(Tl):
    for kk in range(k):
        want[t] += w[t, kk] * x[t] * float(idx[t, kk] + 1)
assert np.allclose(out, want, rtol=1e-5, atol=1e-6), np.abs(out - want).max()
# a rank with a different map must be refused before any exchange
try:
    verify_peers(ExpertSharding.balanced(world, E, [rank + 1] + [1] * (E - 1)) if rank == 1 else sh)
    ok = False
except RuntimeError:
    ok = True
flag = torch.tensor([int(ok)]); dist.all_reduce(flag)
assert flag.item() >= 1
dist.destroy_process_group()
print("OK", rank)
"""


@pytest.mark.parametrize("world", [2, 3])
def test_exchange_layout_agrees_between_ranks_gloo(tmp_path, world):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = str(29000 + (os.getpid() * 7 + world) % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r), str(world)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
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
