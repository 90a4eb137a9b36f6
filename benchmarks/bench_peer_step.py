"""Optimizer step over peer memory: the fused gradient-reduce -> update -> parameter-broadcast kernels in isolation,
with the NVLink bytes they move and the fraction of the link / HBM / tensor-core roofline they reach.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/bench_peer_step.py --optimizer AdamW Muon

Setup: ``--count`` parameters of shape ``--shape`` (fp32) wrapped by ``heavyball_b200.parallel.ddp.wrap(mode="peer")``;
every rank writes random gradients into its gradient slab, then ``--steps`` calls of ``optimizer.step()`` are enqueued
back to back and timed with one pair of CUDA events (barrier + synchronize before; per-step time, maximum over ranks),
so that the host's preparation of a step overlaps the device's execution of the previous one, as in a training loop.  One step = flag barrier, the fused
kernels (each rank loads its share of the gradient from every rank's slab, updates, stores the new parameters into
every rank's slab), flag barrier, clearing of the gradient slab.

Roofline per rank, printed beside the measurement:
* NVLink: bytes loaded from peers and bytes stored to peers (each ``share * (world - 1) * 4``) over the measured
  770 GB/s per direction; loads and stores use opposite directions, so the larger of the two counts;
* HBM: the local traffic of the same kernels (own gradient share, state, parameters) over the measured copy bandwidth;
* tensor cores (Muon): Newton-Schulz FLOPs of the owned matrices over the measured bf16 GEMM rate.
The bound is the largest of the three; ``fraction`` = bound / measured.  ``nccl`` in the output is the same
optimizer on the same shapes after an NCCL all-reduce of the gradient slab (the replicated baseline), for comparison.
"""

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction on this pool


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    except (OSError, ValueError):
        return 6650.0, 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizer", nargs="+", default=["AdamW", "Muon"])
    ap.add_argument("--shape", type=int, nargs=2, default=[2048, 2048])
    ap.add_argument("--count", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--breakdown", action="store_true", help="time barrier / kernels / barrier separately (peer arm)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import heavyball_b200 as hb
    from heavyball_b200.parallel import ddp

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    rank, world = dist.get_rank(), dist.get_world_size()
    hbm_gbs, gemm_tflops, origin = _peaks()
    rows, cols = args.shape
    numel = rows * cols * args.count

    def measure(name, mode):
        torch.manual_seed(0)
        holder = torch.nn.Module()
        holder.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(rows, cols, device=device)) for _ in range(args.count)])
        opt = getattr(hb, name)(holder.parameters(), lr=1e-3)
        wrapped = ddp.wrap(holder, opt, mode="peer") if mode == "peer" else None
        gen = torch.Generator(device=device).manual_seed(1 + rank)
        grads = [torch.randn(rows, cols, device=device, generator=gen) * 0.01 for _ in range(args.count)]

        def fill():
            for p, g in zip(holder.ps, grads):
                if p.grad is None:
                    p.grad = g.clone()
                else:
                    p.grad.copy_(g)

        def one_step():
            if mode == "nccl":  # replicated baseline: average the gradients, every rank updates everything
                flat = torch._utils._flatten_dense_tensors([p.grad for p in holder.ps])
                dist.all_reduce(flat, op=dist.ReduceOp.AVG)
                for p, g in zip(holder.ps, torch._utils._unflatten_dense_tensors(flat, [p.grad for p in holder.ps])):
                    p.grad.copy_(g)
            opt.step()

        for _ in range(args.warmup):
            fill()
            one_step()
        parts = []
        if mode == "peer" and args.breakdown:  # the three parts of one isolated peer step, device and host side
            for _ in range(5):
                fill()
                torch.cuda.synchronize()
                dist.barrier()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                ev[0].record()
                h0 = time.perf_counter()
                wrapped.peer.begin_step()
                ev[1].record()
                h1 = time.perf_counter()
                type(opt).step(opt)  # the class's own step: the instance attribute is the wrapped one
                ev[2].record()
                h2 = time.perf_counter()
                wrapped.peer.end_step()
                ev[3].record()
                h3 = time.perf_counter()
                torch.cuda.synchronize()
                parts.append((ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]), ev[2].elapsed_time(ev[3]),
                              (h1 - h0) * 1e3, (h2 - h1) * 1e3, (h3 - h2) * 1e3))
        # steady state, as inside a training loop: steps are enqueued back to back, so the host's preparation of a
        # step overlaps the device's execution of the previous one (the gradients are whatever the last step left:
        # the traffic does not depend on their values)
        if hasattr(opt, "consume_grad"):
            opt.consume_grad = False  # gradients stay in place between the back-to-back steps
        fill()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            one_step()
        e1.record()
        torch.cuda.synchronize()
        times = [e0.elapsed_time(e1) / args.steps]
        if wrapped is not None and hasattr(wrapped, "peer"):
            wrapped.peer.check()
        hb.ops.check_status()
        if parts and rank == 0:
            med = [statistics.median(x) for x in zip(*parts)]
            print(f"{name} rank 0, one isolated step, device ms: begin barrier {med[0]:.3f}, kernels {med[1]:.3f}, end barrier + "
                  f"clear {med[2]:.3f}; host enqueue ms: {med[3]:.3f}, {med[4]:.3f}, {med[5]:.3f}", flush=True)
        t = torch.tensor([statistics.median(times)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for name in args.optimizer:
        peer_ms = measure(name, "peer")
        nccl_ms = measure(name, "nccl")
        share = numel / world  # elements (AdamW) or elements of owned matrices (Muon) per rank
        link_bytes = share * (world - 1) * 4  # loaded from peers; the same amount is stored to peers
        link_ms = link_bytes / (NVLINK_GBS * 1e9) * 1e3
        if name == "AdamW":
            local_bytes = share * 4 * (1 + 2 + 1 + 2 + 1)  # own gradient share, m and v read, parameter read, m and v, parameter written
            flops = 0.0
        else:
            local_bytes = share * 4 * (1 + 1 + 1 + 1 + 1) + share * 2 * 4  # gradient, momentum r/w, parameter r/w, bf16 X and X^T
            m, n = min(rows, cols), max(rows, cols)
            per_matrix = 5 * (m * m * n + m * m * m + 2 * m * m * n)  # upper-triangular Gram and polynomial, full apply; 2 flop/MAC folded in
            flops = per_matrix * args.count / world
        hbm_ms = local_bytes / (hbm_gbs * 1e9) * 1e3
        mma_ms = flops / (gemm_tflops * 1e12) * 1e3
        bound = max(link_ms, hbm_ms, mma_ms)
        if rank == 0:
            print(json.dumps({
                "optimizer": name, "world": world, "params": numel, "peer_step_ms": peer_ms, "nccl_replicated_step_ms": nccl_ms,
                "nvlink_bytes_each_way_per_rank": link_bytes, "roofline_ms": {"nvlink": link_ms, "hbm": hbm_ms, "tensor": mma_ms},
                "bound_ms": bound, "fraction_of_bound": bound / peer_ms, "peaks": origin,
            }))  # fmt: skip
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
