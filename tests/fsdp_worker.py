"""Worker for the FSDP tests (2+ gloo ranks on CPU, or NCCL ranks on GPUs when launched there).

Every rank trains the same small model on the same batch, once un-sharded in a single process (the
oracle, computed by every rank for simplicity) and once wrapped in ``FullyShardedDataParallel`` with
``use_orig_params=True`` (or, with a trailing ``fsdp2`` argument, sharded by ``fully_shard``); parameters gathered from the sharded run must match the oracle.
"""

import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import heavyball_b200 as hb  # noqa: E402


def make_model(width, depth, seed=0, norm=False):
    torch.manual_seed(seed)
    layers = []
    for _ in range(depth):
        if norm:
            layers.append(nn.LayerNorm(width))
        layers += [nn.Linear(width, width, bias=True), nn.Tanh()]
    return nn.Sequential(*layers, nn.Linear(width, 4))


def train(model, opt, steps, x, y):
    for _ in range(steps):
        loss = nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
    return model


def main():
    name, width, depth, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    tol = float(sys.argv[5]) if len(sys.argv) > 5 else 1e-6
    norm = len(sys.argv) > 6 and sys.argv[6] == "norm"
    fsdp2 = len(sys.argv) > 7 and sys.argv[7] == "fsdp2"
    use_cuda = torch.cuda.is_available() and os.environ.get("HB_TEST_CPU") != "1"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if use_cuda:
        torch.cuda.set_device(rank % torch.cuda.device_count())
        device = torch.device("cuda", rank % torch.cuda.device_count())
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    cls = getattr(hb, name)
    torch.manual_seed(1)
    x = torch.randn(16, width, device=device)
    y = torch.randn(16, 4, device=device)

    ref = make_model(width, depth, norm=norm).to(device)
    torch.manual_seed(7)
    train(ref, cls(ref.parameters(), lr=1e-2), steps, x, y)
    want = torch.cat([p.detach().flatten() for p in ref.parameters()])

    model = make_model(width, depth, norm=norm).to(device)
    if fsdp2:  # fully_shard: DTensor parameters, the optimizer works on their local rows
        from heavyball_b200.parallel import fsdp as hb_fsdp

        fsdp = hb_fsdp.shard(model)
        torch.manual_seed(7)
        opt = cls(fsdp.parameters(), lr=1e-2)
        train(fsdp, opt, steps, x, y)
        got = torch.cat([p.full_tensor().detach().flatten() for p in fsdp.parameters()])
    else:
        fsdp = FSDP(model, use_orig_params=True, device_id=device if use_cuda else None)
        torch.manual_seed(7)
        opt = cls(fsdp.parameters(), lr=1e-2)
        train(fsdp, opt, steps, x, y)
        with FSDP.summon_full_params(fsdp):
            got = torch.cat([p.detach().flatten() for p in fsdp.parameters()])
    movers = [pl.mover for plans in getattr(opt, "_fsdp_plans", {}).values() for pl in plans if pl.mover]
    for mover in movers:
        mover.check()  # no bounded wait of the peer-memory exchange expired
    want_peer = use_cuda and os.environ.get("HB200_FSDP_PEER", "1") != "0" and getattr(opt, "_needs_gather", False)
    if want_peer and not movers:
        print("RESULT peer-memory exchange was expected but the collective path ran")
        sys.exit(1)
    err = (got - want).abs().max().item()
    ok = err <= tol * max(1.0, want.abs().max().item())
    if rank == 0:
        print(f"RESULT {name} width={width} max_err={err:.3e} ok={ok}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
