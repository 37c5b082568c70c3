"""Worker of the multi-GPU expert-parallel parity test (launched by torch.distributed.run, one
rank per GPU).  Every rank runs the expert-parallel block call on its token shard; rank 0 checks the
gathered output against the CPU oracle (routing exact, rel-L2 <= 1e-2) and against the single-GPU
semantics the call promises."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from speedycolibri_b200 import backend, synth  # noqa: E402
from speedycolibri_b200.cluster import ExpertSharding, ShardedMoe  # noqa: E402
from speedycolibri_b200.configs import CONFIGS  # noqa: E402
from speedycolibri_b200.moe import Config  # noqa: E402
from tests.helpers import host_layer, rel_l2, upload_layer  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend.init([local])
    for name, T, balanced, transport in (("tiny_sig", 40 * world, False, "direct"), ("mid", 256 * world, False, "direct"),
                                         ("tiny_zipf", 64 * world, True, "direct"), ("mid", 256 * world, True, "nccl")):
        os.environ["COLI_EP_TRANSPORT"] = transport  # read when the handle's expert-parallel state is created
        shape = CONFIGS[name].with_tokens(T)
        L, packed = host_layer(shape)
        x_all = synth.host_tokens(shape, T)
        want = L.moe_block(x_all)
        if balanced:  # LPT map from the (known) load, as crates/colibri-cluster/src/sharding.rs:87-109
            sharding = ExpertSharding.balanced(world, shape.E, np.bincount(want["idx"].reshape(-1), minlength=shape.E).tolist())
        else:
            sharding = ExpertSharding.new(world, shape.E)
        layer = upload_layer(shape, packed, device=local, local=set(sharding.local_experts(rank)))
        sm = ShardedMoe(Config.from_shape(shape), layer, sharding, T, local)
        # ragged shards: the last rank holds fewer tokens, rank 0 the difference
        cut = [0] + [min(T, (r + 1) * (T // world) + (3 if r + 1 < world else 0)) for r in range(world)]
        cut[-1] = T
        x = torch.from_numpy(x_all[cut[rank]:cut[rank + 1]].view(np.int16)).cuda().view(torch.bfloat16)
        for rep in range(2):
            out = sm(x)
        sm.block.check()
        idx, w = sm.block.last_routing(x.shape[0])
        assert np.array_equal(idx, want["idx"][cut[rank]:cut[rank + 1]]), "routing indices differ from the oracle"
        assert np.array_equal(w.view(np.uint32), want["w"][cut[rank]:cut[rank + 1]].view(np.uint32)), "routing weights differ"
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        err = rel_l2(got, want["out"][cut[rank]:cut[rank + 1]])
        errs = [None] * world
        dist.all_gather_object(errs, err)
        tab = sm.block.ep_last_counts()
        assert tab[:, 1, :].sum() == T * shape.k
        if rank == 0:
            assert max(errs) <= 1e-2, (name, errs)
            print(f"EP_OK {name} {transport} world={world} rel_l2={max(errs):.2e} rows_per_rank={tab[:, 1, :].sum(axis=0).tolist()}", flush=True)
        sm.close()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
