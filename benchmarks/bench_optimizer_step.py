"""Optimizer ``step()`` latency on pre-filled gradients (no forward / backward).

Protocol follows the reference's latency benchmark (``benchmarks/bench_optimizer_step.py:37-81``):
``--count`` parameters of shape ``--shape``, gradients filled once and kept (``consume_grad=False``),
warm-up steps, then windows of steps timed between device synchronisations; the median window is
reported in microseconds per step.  Here each window is timed twice: on the device with CUDA events
and on the host (enqueue time only), which separates kernel time from launch overhead.

    python benchmarks/bench_optimizer_step.py --impl ours --optimizer AdamW Muon --dtype float32
    python benchmarks/bench_optimizer_step.py --impl reference ...   # unmodified reference from baseline/_ref
    python benchmarks/bench_optimizer_step.py --impl torch ...       # torch.optim.AdamW only
"""

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--optimizer", nargs="+", default=["AdamW", "Muon"])
    ap.add_argument("--shape", type=int, nargs="+", default=[2048, 2048])
    ap.add_argument("--count", type=int, default=32)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--windows", type=int, default=6)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--kwargs", default="{}", help="JSON dict of extra optimizer kwargs")
    ap.add_argument("--compile-mode", default=None,
                    help="reference arm only: value for heavyball.utils.compile_mode ('none' = eager); default = stock")
    ap.add_argument("--profile", action="store_true", help="print a torch.profiler table of a few steps (ours / reference)")
    args = ap.parse_args()

    import torch

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import heavyball as lib

        if args.compile_mode is not None:
            lib.utils.compile_mode = None if args.compile_mode.lower() == "none" else args.compile_mode
    elif args.impl == "ours":
        sys.path.insert(0, ROOT)
        import heavyball_b200 as lib
    else:
        lib = torch.optim
    dtype = getattr(torch, args.dtype)
    extra = json.loads(args.kwargs)
    for name in args.optimizer:
        torch.manual_seed(0)
        params = [torch.nn.Parameter(torch.randn(*args.shape, device="cuda", dtype=dtype)) for _ in range(args.count)]
        for p in params:
            p.grad = torch.randn_like(p) * 0.01
        kw = dict(extra)
        if args.impl != "torch":
            kw["consume_grad"] = False
        opt = getattr(lib, name)(params, **kw)
        for _ in range(args.warmup):
            opt.step()
        torch.cuda.synchronize()
        if args.profile:
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
                for _ in range(4):
                    opt.step()
                torch.cuda.synchronize()
            print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=18, max_name_column_width=60))
            print(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=12, max_name_column_width=60))
        dev_us, host_us = [], []
        for _ in range(args.windows):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e0.record()
            for _ in range(args.steps):
                opt.step()
            e1.record()
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            dev_us.append(e0.elapsed_time(e1) * 1e3 / args.steps)
            host_us.append((t1 - t0) * 1e6 / args.steps)
        numel = sum(p.numel() for p in params)
        print(json.dumps({
            "impl": args.impl, "optimizer": name, "kwargs": extra, "shape": args.shape, "count": args.count,
            "dtype": args.dtype, "params": numel, "device_us_per_step": statistics.median(dev_us),
            "host_enqueue_us_per_step": statistics.median(host_us),
        }))


if __name__ == "__main__":
    main()
