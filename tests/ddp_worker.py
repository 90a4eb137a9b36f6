"""Worker for the multi-GPU data-parallel test (launched by ``torch.distributed.run``).

Trains a small GPT for a few steps on rank-specific data: with the peer-memory scheme and with
``DistributedDataParallel`` + replicated optimizer.  Checks that (a) replicas are bit-identical under the
peer scheme, (b) both schemes agree to rounding noise, (c) no bounded wait expired, (d) under bf16 autocast the
peer scheme gives the same parameters whether forward and backward are launched kernel by kernel or replayed
from CUDA graphs, (e) after ``consolidate_state`` every rank holds the complete optimizer state, equal to the
replicated run's.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import heavyball_b200 as hb  # noqa: E402
from heavyball_b200.models import GPT, GPTConfig, graph_forward_backward, split_param_groups  # noqa: E402
from heavyball_b200.parallel import ddp  # noqa: E402


def run(mode, steps, rank, world, device, autocast=False, graphs=False):
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=2, n_head=4, d_model=256, vocab_size=512, seq_len=64)).to(device)
    mats, rest = split_param_groups(model)
    opt = hb.SplitOpt([
        {"params": mats, "optimizer": hb.Muon, "lr": 0.02, "weight_decay": 0.01},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-3},
    ])
    wrapped = ddp.wrap(model, opt, mode=mode)
    gen = torch.Generator().manual_seed(100 + rank)
    if graphs:
        example = torch.randint(0, 512, (4, 65), generator=torch.Generator().manual_seed(5)).to(device)  # own generator:
        # the default one seeds the optimizer's stochastic rounding and must see the same draws in both runs
        graph_forward_backward(model, (example[:, :-1], example[:, 1:]))
    losses = []
    for _ in range(steps):
        tokens = torch.randint(0, 512, (4, 65), generator=gen).to(device)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast, cache_enabled=False):
            loss = wrapped(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.detach().clone())
    if hasattr(wrapped, "peer"):
        wrapped.peer.check()
        wrapped.peer.consolidate_state()
    hb.ops.check_status()
    flat = torch.cat([p.detach().flatten().float() for p in model.parameters()])
    state = []
    for inner in opt.optimizers if hasattr(opt, "optimizers") else [opt]:
        for p in model.parameters():
            if p in inner.state:
                state += [t.detach().flatten().float() for t in ddp.PeerContext._state_tensors(inner, p)]
    return flat, torch.stack(losses), torch.cat(state)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    steps = 4
    peer_flat, peer_loss, peer_state = run("peer", steps, rank, world, device)
    nccl_flat, nccl_loss, nccl_state = run("nccl", steps, rank, world, device)
    amp_flat, amp_loss, _ = run("peer", steps, rank, world, device, autocast=True)
    graph_flat, graph_loss, _ = run("peer", steps, rank, world, device, autocast=True, graphs=True)
    # after consolidation every rank holds the whole optimizer state, and it is the replicated run's state
    states = [torch.empty_like(peer_state) for _ in range(world)]
    dist.all_gather(states, peer_state)
    state_identical = all(torch.equal(states[0], s) for s in states)
    state_rms = ((peer_state - nccl_state).square().mean().sqrt() / nccl_state.square().mean().sqrt()).item()
    graph_rms = ((amp_flat - graph_flat).square().mean().sqrt() / amp_flat.square().mean().sqrt()).item()

    gathered = [torch.empty_like(peer_flat) for _ in range(world)]
    dist.all_gather(gathered, peer_flat)
    identical = all(torch.equal(gathered[0], g) for g in gathered)
    diff = (peer_flat - nccl_flat).abs().max().item()
    scale = nccl_flat.abs().max().item()
    rms = ((peer_flat - nccl_flat).square().mean().sqrt() / nccl_flat.square().mean().sqrt()).item()
    if rank == 0:
        print(f"multimem={os.environ.get('HB200_PEER_MULTIMEM', '1')} ", end="")
        print(f"RESULT identical={identical} max_abs_diff={diff:.3e} max_abs={scale:.3e} rel_rms={rms:.3e} "
              f"loss_peer={peer_loss.tolist()} loss_nccl={nccl_loss.tolist()} graph_rel_rms={graph_rms:.3e} "
              f"loss_amp={amp_loss.tolist()} loss_graph={graph_loss.tolist()} state_identical={state_identical} "
              f"state_rel_rms={state_rms:.3e}")
    ok = identical and rms < 2e-2 and graph_rms < 2e-2 and state_identical and state_rms < 2e-2
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
