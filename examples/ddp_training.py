"""Data-parallel training of a small GPT with SplitOpt(Muon, AdamW).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/ddp_training.py [--mode nccl]

``--mode peer`` (default) uses symmetric-memory slabs: the optimizer kernels reduce gradients on load and
broadcast parameters on store, and every matrix is orthogonalised by one owner rank.  ``--mode nccl`` is the
classic path (``DistributedDataParallel`` + replicated optimizer).  Data is synthetic.
"""

import argparse
import os

import torch
import torch.distributed as dist

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb
from heavyball_b200.models import GPT, GPTConfig, split_param_groups
from heavyball_b200.parallel import ddp


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--save", default=None, help="write a checkpoint (model + optimizer state) here at the end")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=4, n_head=8, d_model=512, vocab_size=8192, seq_len=256)).to(device)
    mats, rest = split_param_groups(model)
    opt = hb.SplitOpt([
        {"params": mats, "optimizer": hb.Muon, "lr": 0.02, "weight_decay": 0.01},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-4},
    ])
    net = ddp.wrap(model, opt, mode=args.mode)
    gen = torch.Generator().manual_seed(dist.get_rank())
    for step in range(args.steps):
        tokens = torch.randint(0, 8192, (8, 257), generator=gen).to(device)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        if step % 10 == 0 and dist.get_rank() == 0:
            print(f"step {step:4d}  loss {loss.item():.4f}")
    if hasattr(net, "peer"):
        net.peer.check()
        net.peer.consolidate_state()  # collective: optimizer state is partitioned across ranks until now
    if dist.get_rank() == 0 and args.save:
        torch.save({"model": model.state_dict(), "optimizer": opt.state_dict()}, args.save)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
