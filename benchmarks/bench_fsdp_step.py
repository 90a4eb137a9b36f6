"""Optimizer ``step()`` latency under FSDP1 (flat parameters, ``use_orig_params=True``) with an optimizer that needs
whole matrices (Muon by default), i.e. the owner-repartition path: shards and gradient shards travel to an owner
rank, the owner updates the full matrix, the updated shards travel back.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/bench_fsdp_step.py --impl ours --optimizer Muon --layers 12 --width 1024
    ... --impl reference         # the unmodified reference from baseline/_ref (eager: --compile-mode none)

A stack of ``--layers`` square ``Linear(width, width)`` layers stands in for a transformer's matrices.  Gradients are
produced by one real forward/backward per step (FSDP needs its own reduce-scatter to run); only ``optimizer.step()``
is timed, with CUDA events, and the maximum over ranks of the median step is reported.  The reference exchanges
split sizes, headers and payload per 32 MiB bucket every step (nine collectives and four host synchronisations);
this framework plans once and issues one ``all_to_all_single`` per dtype each way
(``heavyball_b200/parallel/fsdp.py``; reference: ``heavyball/chainable.py:2009-2213``).
"""

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--optimizer", default="Muon")
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--kwargs", default="{}")
    ap.add_argument("--compile-mode", default=None, help="reference arm: heavyball.utils.compile_mode ('none' = eager)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import heavyball as lib

        if args.compile_mode is not None:
            lib.utils.compile_mode = None if args.compile_mode.lower() == "none" else args.compile_mode
    else:
        sys.path.insert(0, ROOT)
        import heavyball_b200 as lib

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    rank, world = dist.get_rank(), dist.get_world_size()

    torch.manual_seed(0)
    layers = []
    for _ in range(args.layers):
        layers += [nn.Linear(args.width, args.width, bias=False), nn.Tanh()]
    model = FSDP(nn.Sequential(*layers).to(device), use_orig_params=True, device_id=device)
    opt = getattr(lib, args.optimizer)(model.parameters(), lr=1e-3, **json.loads(args.kwargs))
    x = torch.randn(args.batch, args.width, device=device)

    times = []
    for i in range(args.warmup + args.steps):
        model(x).square().mean().backward()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        opt.zero_grad()
        if i >= args.warmup:
            times.append(e0.elapsed_time(e1))
    med = torch.tensor([statistics.median(times)], dtype=torch.float64, device=device)
    dist.all_reduce(med, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "impl": args.impl, "optimizer": args.optimizer, "world": world, "layers": args.layers, "width": args.width,
            "params": args.layers * args.width * args.width, "optimizer_step_ms_median_max_over_ranks": float(med.item()),
            "min_ms": min(times), "max_ms": max(times),
        }))  # fmt: skip
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
