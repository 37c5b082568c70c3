"""Worker of the multi-GPU expert-parallel parity test (launched by torch.distributed.run, one
rank per GPU).  Every rank runs cluster.moe_sharded on its token shard; rank 0 checks the gathered
output against the CPU oracle and against the reference's sharded == single-node property."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from speedycolibri_b200 import backend, synth  # noqa: E402
from speedycolibri_b200.cluster import ExpertSharding, moe_sharded, verify_peers  # noqa: E402
from speedycolibri_b200.configs import CONFIGS  # noqa: E402
from speedycolibri_b200.moe import Config, MoeBlock  # noqa: E402
from tests.helpers import host_layer, rel_l2, upload_layer  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend.init([local])
    for name, T, balanced in (("tiny_sig", 40 * world, False), ("mid", 256 * world, False), ("tiny_zipf", 64 * world, True)):
        shape = CONFIGS[name].with_tokens(T)
        L, packed = host_layer(shape)
        x_all = synth.host_tokens(shape, T)
        if balanced:  # LPT map from the (known) load, as crates/colibri-cluster/src/sharding.rs:87-109
            idx, _ = L.route_tokens(x_all)
            sharding = ExpertSharding.balanced(world, shape.E, np.bincount(idx.reshape(-1), minlength=shape.E).tolist())
        else:
            sharding = ExpertSharding.new(world, shape.E)
        verify_peers(sharding)
        layer = upload_layer(shape, packed, device=local, local=set(sharding.local_experts(rank)))
        blk = MoeBlock(Config.from_shape(shape), layer, T, device=local, ep_rank=rank, ep_world=world,
                       expert_owner=sharding.owner_table() if balanced else None)
        Tl = T // world
        x = torch.from_numpy(x_all[rank * Tl:(rank + 1) * Tl].view(np.int16)).cuda().view(torch.bfloat16)
        for rep in range(2):
            out = moe_sharded(blk, sharding, x)
        blk.check()
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(outs, out)
        if rank == 0:
            got = torch.cat(outs).view(torch.int16).cpu().numpy().view(np.uint16)
            want = L.moe_block(x_all, world=world, owner=np.array(sharding.owner_table(), np.int32) if balanced else None)
            err = rel_l2(got, want["out"])
            assert err <= 1e-2, (name, err)
            print(f"EP_OK {name} world={world} rel_l2={err:.2e}", flush=True)
        blk.close()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
