"""Headline benchmark: training throughput (tokens/s) and optimizer step time of a GPT-2-small-shaped
decoder trained with SplitOpt(Muon lr 0.02 on the 2-D block weights, AdamW lr 3e-4 on the rest),
bf16 autocast over fp32 master weights, 16 sequences x 1024 tokens per GPU, synthetic token ids.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks, inputs
pre-staged on the GPU); ``e2e.value`` times the same steps through the public API including the
pinned host->device copy of every step's tokens and the device->host read of its loss.

``--impl reference`` runs the unmodified reference package installed under ``baseline/_ref`` (its own
optimizers and stock compile path, ``torch.nn`` DDP, a plain ``torch.nn`` model) for the same metric.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PUBLISHED_BASELINE = None  # the reference publishes no tokens/s figure for this config

CONFIGS = {
    "gpt2-small": dict(n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024, seqs_per_gpu=16),
    "gpt2-tiny": dict(n_layer=2, n_head=4, d_model=256, vocab_size=4096, seq_len=256, seqs_per_gpu=4),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--graphs", default="auto", choices=["auto", "on", "off"],
                    help="our arm: replay forward and backward from CUDA graphs (auto = on, falling back to eager "
                         "launches if capture fails)")
    ap.add_argument("--cuda-profiler", action="store_true",
                    help="bracket the device-timed steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--no-clocks", action="store_true", help="do not run the nvidia-smi clock sampler (diagnostics)")
    ap.add_argument("--trace-steps", action="store_true", help="also print every timed step's device time to stderr")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gpt2-small", choices=sorted(CONFIGS))
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end phase")
    ap.add_argument("--ddp-mode", default="peer", choices=["peer", "nccl"], help="gradient path of the 'ours' arm")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.

    nvidia-smi is started before the warm-up steps (its start-up initialises NVML on every GPU of the node and
    stalls running kernels for up to a second, which must not land in the timed region); samples carry
    timestamps and only those taken between ``begin()`` and ``stop()`` are summarised."""

    FIELDS = (
        "timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, device_index):
        self.proc, self.index, self.t_begin = None, device_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self.proc = None
            return
        import threading

        self.lines = []
        self.reader = threading.Thread(target=lambda: self.lines.extend(iter(self.proc.stdout.readline, "")), daemon=True)
        self.reader.start()
        deadline = time.time() + 5.0  # first sample printed = NVML start-up is over
        while not self.lines and time.time() < deadline and self.proc.poll() is None:
            time.sleep(0.02)

    def begin(self):
        self.t_begin = time.time()

    @staticmethod
    def _stamp(text):
        import datetime

        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        t_end = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)  # let the sample that covers the end of the region be written
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            self.proc.wait()
        self.reader.join(timeout=2)
        rows = []
        for line in list(self.lines):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                rows.append((self._stamp(parts[0]), float(parts[2]), float(parts[3]), parts[5:9]))
            except ValueError:
                continue
        t0 = self.t_begin if self.t_begin is not None else 0.0
        inside = [r for r in rows if r[0] is not None and t0 <= r[0] <= t_end + 0.1]
        if not inside:  # region shorter than the sampling period: take the samples nearest to it
            inside = [r for r in rows if r[0] is None or r[0] >= t0 - 0.25][:3] or rows[-3:]
        clocks = sorted(r[1] for r in inside)
        reasons = {name for r in inside for name, val in zip(self.NAMES, r[3]) if val.lower().startswith("active")}
        return {
            "sm_mhz": clocks[len(clocks) // 2] if clocks else None,
            "sm_max_mhz": max((r[2] for r in inside), default=None),
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


def build_ours(cfg, device):
    import heavyball_b200 as hb
    from heavyball_b200.models import GPT, GPTConfig, split_param_groups

    model = GPT(GPTConfig(cfg["n_layer"], cfg["n_head"], cfg["d_model"], 0, cfg["vocab_size"], cfg["seq_len"])).to(device)
    mats, rest = split_param_groups(model)
    opt = hb.SplitOpt([
        {"params": mats, "optimizer": hb.Muon, "lr": 0.02},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-4},
    ])
    return model, opt


def build_reference(cfg, device):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import heavyball
    from ref_model import RefGPT, split

    mode = os.environ.get("HB_REF_COMPILE_MODE")  # unset = the reference's stock setting
    if mode is not None:
        heavyball.utils.compile_mode = None if mode in ("", "none") else mode
    model = RefGPT(cfg["n_layer"], cfg["n_head"], cfg["d_model"], cfg["vocab_size"], cfg["seq_len"]).to(device)
    mats, rest = split(model)
    opt = heavyball.SplitOpt([
        {"params": mats, "optimizer": heavyball.Muon, "lr": 0.02},
        {"params": rest, "optimizer": heavyball.AdamW, "lr": 3e-4},
    ])
    return model, opt


def main():
    args = parse()
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "heavyball")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    cfg = CONFIGS[args.config]
    torch.manual_seed(0)
    model, opt = (build_ours if args.impl == "ours" else build_reference)(cfg, device)
    launches = None
    if args.impl == "ours":
        from heavyball_b200 import ops

        launches = ops.launch_counter
    if world > 1:
        if args.impl == "ours":
            from heavyball_b200.parallel import ddp as hb_ddp

            train_model = hb_ddp.wrap(model, opt, mode=args.ddp_mode)
        else:
            from torch.nn.parallel import DistributedDataParallel

            train_model = DistributedDataParallel(model, device_ids=[local])
    else:
        train_model = model

    B, T, V = cfg["seqs_per_gpu"], cfg["seq_len"], cfg["vocab_size"]
    n_host = 8
    gen = torch.Generator().manual_seed(1234 + rank)
    host_tokens = [torch.randint(0, V, (B, T + 1), generator=gen).pin_memory() for _ in range(n_host)]
    dev_tokens = [t.to(device) for t in host_tokens]

    graphed = False

    def train_step(tokens):
        with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=not graphed):
            loss = train_model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    launches_per_step = None
    if args.impl == "ours":
        # two eager steps: create the optimizer state, then count this repository's kernel launches per step (inside
        # CUDA graphs the same kernels run, but the Python-side counter only sees them at capture time)
        train_step(dev_tokens[0])  # first step: state initialisation takes its own path
        launches.reset()
        train_step(dev_tokens[1 % n_host])
        launches_per_step = launches.count
        if args.graphs != "off":
            try:
                from heavyball_b200.models import graph_forward_backward

                graph_forward_backward(model, (dev_tokens[0][:, :-1], dev_tokens[0][:, 1:]))
                graphed = True
            except Exception as err:  # noqa: BLE001
                if args.graphs == "on":
                    raise
                print(f"graph capture failed ({type(err).__name__}: {err}); running eager launches", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    if rank == 0 and not args.no_clocks:
        sampler.start()
    for i in range(args.warmup):
        train_step(dev_tokens[i % n_host])
    # Python's cyclic collector pauses one rank for milliseconds at unpredictable steps, and in data-parallel runs
    # every rank then waits for it: collect now, keep it off while timing (both arms)
    import gc

    gc.collect()
    gc.disable()
    barrier()

    # ---- phase 1: device-timed, inputs already on the GPU
    if launches is not None:
        launches.reset()
    opt_ms = []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.begin()
    if args.cuda_profiler:
        torch.cuda.profiler.start()
    start.record()
    last = None
    marks = []
    for i in range(args.steps):
        last = train_step(dev_tokens[i % n_host])
        if args.trace_steps:
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record()
    stop.record()
    last = last.detach().clone()  # under CUDA graphs the returned loss is a static buffer that later replays overwrite
    barrier()
    if args.cuda_profiler:
        torch.cuda.profiler.stop()
    if marks:
        per_step = [a.elapsed_time(b) for a, b in zip([start] + marks[:-1], marks)]
        print(f"rank {rank} step ms: " + " ".join(f"{t:.1f}" for t in per_step), file=sys.stderr)
    n_launch = launches_per_step * args.steps if launches_per_step is not None else None
    clocks = sampler.stop() if (rank == 0 and not args.no_clocks) else None
    step_ms = max_over_ranks(start.elapsed_time(stop) / args.steps)

    # ---- optimizer step alone (same state, gradients from one backward), device-timed
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(min(args.steps, 10)):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = train_model(dev_tokens[i % n_host][:, :-1], dev_tokens[i % n_host][:, 1:])
        loss.backward()
        torch.cuda.synchronize()
        e0.record()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        opt.zero_grad(set_to_none=True)
        opt_ms.append(e0.elapsed_time(e1))
    opt_ms.sort()
    opt_step_ms = max_over_ranks(opt_ms[len(opt_ms) // 2])

    # ---- phase 2: end to end through the public API: every step copies its tokens from pinned host memory and
    # copies its loss back into pinned host memory.  The loss copy is asynchronous and its value is consumed
    # one step later (as a training loop that logs its loss does), so the host stays at most one step ahead of
    # the device instead of draining the queue every step.
    e2e = None
    if not args.no_e2e:
        loss_host = torch.empty(args.steps, dtype=torch.float32).pin_memory()
        copied = [torch.cuda.Event() for _ in range(args.steps)]
        seen = []
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            tokens = host_tokens[i % n_host].to(device, non_blocking=True)
            loss = train_step(tokens)
            loss_host[i : i + 1].copy_(loss.detach().float().reshape(1), non_blocking=True)
            copied[i].record()
            if i:
                copied[i - 1].synchronize()
                seen.append(float(loss_host[i - 1]))
        copied[-1].synchronize()
        seen.append(float(loss_host[args.steps - 1]))
        barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps)
        e2e = {
            "value": B * T * world / (e2e_ms * 1e-3),
            "unit": "tokens/s",
            "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": host_tokens[0].numel() * host_tokens[0].element_size(),
            "d2h_bytes_per_step": 4,
            "loss_readback": "async copy into pinned memory every step, value consumed one step later",
            "losses_finite": all(v == v and abs(v) != float("inf") for v in seen),
        }

    gc.enable()
    if args.impl == "ours":
        from heavyball_b200 import ops

        ops.check_status()
        if hasattr(train_model, "peer"):
            train_model.peer.check()
    if rank == 0:
        value = B * T * world / (step_ms * 1e-3)
        out = {
            "metric": "train tokens/s (GPT-2-small, SplitOpt Muon+AdamW); optimizer step ms in 'optimizer_step_ms'",
            "impl": args.impl,
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": step_ms,
            "optimizer_step_ms": opt_step_ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": (value / PUBLISHED_BASELINE) if PUBLISHED_BASELINE else None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "config": {
                "model": args.config, "global_batch": B * world, "seq_len": T, "parallelism": f"dp{world}",
                "gradient_path": (args.ddp_mode if (args.impl == "ours" and world > 1) else ("nccl-ddp" if world > 1 else "none")),
                "optimizer": "SplitOpt(Muon lr=0.02 NS5 on 2-D block weights, AdamW lr=3e-4 on the rest)",
                "precision": "bf16 autocast, fp32 master weights and optimizer state",
                "cuda_graphs": "forward and backward replayed from CUDA graphs, optimizer launched eagerly" if graphed else "none",
                "l2": "per-step working set (activations, 124M fp32 params + state) exceeds the 126 MB L2",
            },
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": n_launch,
            "final_loss": float(last.detach()),
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
