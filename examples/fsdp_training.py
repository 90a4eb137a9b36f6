"""FSDP with a shape-dependent optimizer: flat-parameter sharding (``use_orig_params=True``) or, with ``--fsdp2``,
``fully_shard`` and DTensor parameters.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/fsdp_training.py [--fsdp2]

Every sharded matrix gets an owner rank; its shards and gradient shards travel to the owner, the owner runs
SOAP (or Muon / PSGD) on the full matrix and sends the updated shards back.  Nothing else is needed: the
optimizer detects the sharding on its first step (FSDP1) or reads it off the DTensor placements (FSDP2); on NCCL jobs
the slices move through peer memory (one gather and one scatter launch).  For sharders other than FSDP call
``heavyball_b200.capture_param_shapes(model)`` before wrapping and pass the result as ``orig_shapes=``.
"""

import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb


def main():
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 512), nn.GELU(), nn.Linear(512, 10)).to(device)
    if "--fsdp2" in sys.argv[1:]:
        from heavyball_b200.parallel import fsdp as hb_fsdp

        model = hb_fsdp.shard(model)
    else:
        model = FSDP(model, use_orig_params=True, device_id=device)
    opt = hb.SOAP(model.parameters(), lr=3e-3, precondition_frequency=4)
    gen = torch.Generator().manual_seed(dist.get_rank())
    for step in range(40):
        x = torch.randn(64, 256, generator=gen).to(device)
        y = torch.randint(0, 10, (64,), generator=gen).to(device)
        loss = nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        if step % 10 == 0 and dist.get_rank() == 0:
            print(f"step {step:3d}  loss {loss.item():.4f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
