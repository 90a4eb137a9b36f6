"""Worker for the multi-GPU test of the peer-memory data-parallel step on flagged and second-order chains.

For every variant a small GPT is trained for a few steps on rank-specific data twice: with the peer-memory scheme and
with ``DistributedDataParallel`` + replicated optimizer.  Checked per variant: the peer scheme really planned the
group (no silent fallback to a collective), replicas are bit-identical afterwards, both schemes agree within the noise
the variant's random rounding allows, no bounded wait expired.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import heavyball_b200 as hb  # noqa: E402
from heavyball_b200.models import GPT, GPTConfig, split_param_groups  # noqa: E402
from heavyball_b200.parallel import ddp  # noqa: E402

VARIANTS = {
    "adamw-caution-ecc": (lambda m, r: hb.AdamW(m + r, lr=3e-3, caution=True, ecc="bf16+8"), torch.float32, 3e-2),
    # ADOPT divides by the previous step's second moment: only for the densely updated block weights (embedding rows
    # that were not looked up in the seeding step would divide by eps)
    "adopt": (lambda m, r: hb.SplitOpt([{"params": m, "optimizer": hb.ADOPT, "lr": 1e-3},
                                        {"params": r, "optimizer": hb.AdamW, "lr": 3e-3}]), torch.float32, 2e-2),
    "muon-ecc-mars-caution": (
        lambda m, r: hb.SplitOpt([
            {"params": m, "optimizer": hb.Muon, "lr": 0.02, "ecc": "bf16+8", "param_ecc": "bf16+8", "mars": True, "caution": True},
            {"params": r, "optimizer": hb.AdamW, "lr": 3e-3},
        ]), torch.bfloat16, 5e-2),  # fmt: skip  (param_ecc narrows the block weights to bf16: forward under autocast)
    "psgd": (lambda m, r: hb.PSGDKron(m + r, lr=1e-3, preconditioner_update_probability=0.5), torch.float32, 5e-2),
    "soap": (lambda m, r: hb.SOAP(m + r, lr=3e-3, precondition_frequency=2), torch.float32, 5e-2),
}


def run(variant, mode, steps, rank, device):
    make, dtype, _ = VARIANTS[variant]
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=2, n_head=4, d_model=256, vocab_size=512, seq_len=64)).to(device)
    mats, rest = split_param_groups(model)
    opt = make(mats, rest)
    wrapped = ddp.wrap(model, opt, mode=mode)
    planned = len(wrapped.peer.plans) if hasattr(wrapped, "peer") else 0
    if hasattr(wrapped, "peer") and rank == 0:
        print(f"INFO {variant}: NVSwitch multicast in use = {wrapped.peer.multicast}")
    gen = torch.Generator().manual_seed(100 + rank)
    for _ in range(steps):
        tokens = torch.randint(0, 512, (4, 65), generator=gen).to(device)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16, cache_enabled=False):
            loss = wrapped(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
    if hasattr(wrapped, "peer"):
        wrapped.peer.check()
    hb.ops.check_status()
    return torch.cat([p.detach().flatten().float() for p in model.parameters()]), planned, float(loss)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    names = sys.argv[1:] or list(VARIANTS)
    ok = True
    for name in names:
        peer_flat, planned, peer_loss = run(name, "peer", 5, rank, device)
        nccl_flat, _, nccl_loss = run(name, "nccl", 5, rank, device)
        gathered = [torch.empty_like(peer_flat) for _ in range(world)]
        dist.all_gather(gathered, peer_flat)
        identical = all(torch.equal(gathered[0], g) for g in gathered)
        rms = ((peer_flat - nccl_flat).square().mean().sqrt() / nccl_flat.square().mean().sqrt()).item()
        good = identical and planned > 0 and rms < VARIANTS[name][2] and peer_loss == peer_loss
        ok = ok and good
        if rank == 0:
            print(f"RESULT {name} identical={identical} planned_groups={planned} rel_rms={rms:.3e} "
                  f"loss_peer={peer_loss:.4f} loss_nccl={nccl_loss:.4f} ok={good}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
