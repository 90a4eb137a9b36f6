"""Training-throughput benchmark (tokens/s, step ms, optimizer-step ms) on synthetic token ids.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config NAME]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints one JSON line.

Configurations (``--config``):

``gpt2-small`` (default, the headline)  GPT-2-small decoder, SplitOpt(Muon lr 0.02 on the 2-D block weights, AdamW
    lr 3e-4 on the rest), bf16 autocast over fp32 master weights, 16 x 1024 tokens per GPU, data parallel.
``gpt-350m-psgd``   24-layer / 1024-wide GPT, PSGDKron(preconditioner_update_probability=0.1,
    max_size_triangular=8192, ecc="bf16+8"), 8 x 1024 tokens per GPU, data parallel.
``llama-1.3b-soap``  Llama-style 1.3B, SOAP(lr 3e-3, betas (0.95, 0.95), shampoo_beta 0.95,
    precondition_frequency 10, max_precond_dim 4096), 4 x 2048 tokens per GPU, fully sharded.
``llama3-8b-muon-ecc``  Llama-3-8B shape in bf16, SplitOpt(Muon(ecc, param_ecc = "bf16+8", mars, caution) on block
    weights, AdamW on the rest), 1 x 4096 tokens per GPU, fully sharded.

What is measured, per configuration: ``value`` = tokens/s from ``--windows`` timed windows of exactly ``--steps``
steps each (CUDA events around a window, a barrier and a device synchronisation on both sides, max over ranks, the
median window is reported, inputs already on the GPU); ``optimizer_step_ms`` and ``fwd_bwd_ms`` = the two halves of a
step timed separately; ``e2e`` = the same steps through the public API including the pinned host->device copy of every
step's tokens and the device->host read of its loss.

The default configuration's line also carries ``plain_model`` (this package's optimizers driving the plain ``torch.nn``
model of ``baseline/ref_model.py``, i.e. the optimizer's share of the speed-up with the model held fixed) and
``secondary`` (the other configurations, a few steps each).  Those run as child processes after the headline numbers
are taken, each under a time limit, so a failure there cannot lose the headline.

``--impl reference`` runs the unmodified reference package installed under ``baseline/_ref`` (its own optimizers and
stock compile path, ``torch.nn`` DDP / FSDP, the plain ``torch.nn`` models) for the same metric.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PUBLISHED_BASELINE = None  # the reference publishes no tokens/s figure for these configurations

CONFIGS = {
    "gpt2-small": dict(family="gpt", n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024, seqs_per_gpu=16,
                       optimizer="muon+adamw", parallelism="dp", master="fp32"),
    "gpt2-tiny": dict(family="gpt", n_layer=2, n_head=4, d_model=256, vocab_size=4096, seq_len=256, seqs_per_gpu=4,
                      optimizer="muon+adamw", parallelism="dp", master="fp32"),
    "gpt-350m-psgd": dict(family="gpt", n_layer=24, n_head=16, d_model=1024, vocab_size=50257, seq_len=1024,
                          seqs_per_gpu=8, optimizer="psgd", parallelism="dp", master="fp32"),
    "gpt-tiny-psgd": dict(family="gpt", n_layer=2, n_head=4, d_model=256, vocab_size=4096, seq_len=256, seqs_per_gpu=4,
                          optimizer="psgd", parallelism="dp", master="fp32"),
    "llama-1.3b-soap": dict(family="llama", n_layer=24, n_head=16, n_kv_head=16, d_model=2048, d_ff=5504,
                            vocab_size=32000, seq_len=2048, rope_theta=10000.0, seqs_per_gpu=4, optimizer="soap",
                            parallelism="fsdp", master="fp32"),
    "llama-tiny-soap": dict(family="llama", n_layer=2, n_head=4, n_kv_head=4, d_model=256, d_ff=512, vocab_size=4096,
                            seq_len=256, rope_theta=10000.0, seqs_per_gpu=4, optimizer="soap", parallelism="fsdp",
                            master="fp32"),
    "llama3-8b-muon-ecc": dict(family="llama", n_layer=32, n_head=32, n_kv_head=8, d_model=4096, d_ff=14336,
                               vocab_size=128256, seq_len=4096, rope_theta=500000.0, seqs_per_gpu=1,
                               optimizer="muon-ecc+adamw", parallelism="fsdp", master="bf16"),
    "llama-tiny-muon-ecc": dict(family="llama", n_layer=2, n_head=4, n_kv_head=2, d_model=256, d_ff=512,
                                vocab_size=4096, seq_len=256, rope_theta=500000.0, seqs_per_gpu=2,
                                optimizer="muon-ecc+adamw", parallelism="fsdp", master="bf16"),
}  # fmt: skip
SECONDARY = ("gpt-350m-psgd", "llama-1.3b-soap", "llama3-8b-muon-ecc")
OPTIMIZER_TEXT = {
    "muon+adamw": "SplitOpt(Muon lr=0.02 NS5 on 2-D block weights, AdamW lr=3e-4 on the rest)",
    "psgd": "PSGDKron(preconditioner_update_probability=0.1, max_size_triangular=8192, ecc='bf16+8')",
    "soap": "SOAP(lr=3e-3, betas=(0.95, 0.95), shampoo_beta=0.95, precondition_frequency=10, max_precond_dim=4096)",
    "muon-ecc+adamw": "SplitOpt(Muon lr=0.02 ecc='bf16+8' param_ecc='bf16+8' mars caution on 2-D block weights, "
                      "AdamW lr=3e-4 on the rest)",
}  # fmt: skip
VOCAB_MULTIPLE = 64


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--windows", type=int, default=10, help="timed windows of --steps steps each; the median is reported")
    ap.add_argument("--graphs", default="auto", choices=["auto", "on", "off"],
                    help="our arm: replay forward and backward from CUDA graphs (auto = on, falling back to eager "
                         "launches if capture fails)")
    ap.add_argument("--cuda-profiler", action="store_true",
                    help="bracket the device-timed steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--no-clocks", action="store_true", help="do not run the nvidia-smi clock sampler (diagnostics)")
    ap.add_argument("--trace-steps", action="store_true", help="also print every timed step's device time to stderr")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gpt2-small", choices=sorted(CONFIGS))
    ap.add_argument("--model", default="native", choices=["native", "plain"],
                    help="our arm: this package's model (native) or the plain torch.nn model the reference arm uses")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end phase")
    ap.add_argument("--ddp-mode", default="peer", choices=["peer", "nccl"], help="gradient path of the 'ours' arm")
    ap.add_argument("--secondary", default="auto", choices=["auto", "on", "off"],
                    help="also run the plain-model measurement and the other configurations as child processes "
                         "(auto = only for the default configuration)")
    ap.add_argument("--secondary-steps", type=int, default=4)
    ap.add_argument("--secondary-timeout", type=float, default=600.0, help="seconds per child process")
    ap.add_argument("--secondary-budget", type=float, default=1300.0, help="seconds for all child processes together")
    ap.add_argument("--reference-compile-mode", default=None,
                    help="reference arm: value for heavyball.utils.compile_mode ('none' = eager); default = stock")
    return ap.parse_args(argv)


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


# ---------------------------------------------------------------------------------------- models and optimizers


def vocab_rows(cfg):
    """Embedding / head rows: the GPT vocabularies are rounded up to a multiple of 64 in BOTH arms (same parameter
    shapes for both optimizers); the Llama vocabularies already are multiples of 64."""
    v = cfg["vocab_size"]
    return -(-v // VOCAB_MULTIPLE) * VOCAB_MULTIPLE if cfg["family"] == "gpt" else v


def build_model(cfg, kind, device, dtype):
    """``kind``: "native" = heavyball_b200.models, "plain" = baseline/ref_model.py (torch.nn only)."""
    import torch

    with torch.device(device):
        if kind == "native":
            from heavyball_b200 import models

            if cfg["family"] == "gpt":
                model = models.GPT(models.GPTConfig(cfg["n_layer"], cfg["n_head"], cfg["d_model"], 0, cfg["vocab_size"],
                                                    cfg["seq_len"], vocab_multiple=VOCAB_MULTIPLE))  # fmt: skip
            else:
                model = models.Llama(models.LlamaConfig(cfg["n_layer"], cfg["n_head"], cfg["n_kv_head"], cfg["d_model"],
                                                        cfg["d_ff"], cfg["vocab_size"], cfg["seq_len"], cfg["rope_theta"]))  # fmt: skip
        else:
            if os.path.join(ROOT, "baseline") not in sys.path:
                sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import ref_model

            if cfg["family"] == "gpt":
                model = ref_model.RefGPT(cfg["n_layer"], cfg["n_head"], cfg["d_model"], cfg["vocab_size"], cfg["seq_len"],
                                         vocab_rows=vocab_rows(cfg))  # fmt: skip
            else:
                model = ref_model.RefLlama(cfg["n_layer"], cfg["n_head"], cfg["n_kv_head"], cfg["d_model"], cfg["d_ff"],
                                           cfg["vocab_size"], cfg["seq_len"], cfg["rope_theta"])  # fmt: skip
    if dtype is not None:
        model = model.to(dtype)
    return model


def matrix_names(model):
    """Names of the 2-D weights inside the transformer blocks (decided before any sharding wrapper flattens them)."""
    out = set()
    for name, p in model.named_parameters():
        if p.ndim >= 2 and (name.startswith(("blocks.", "layers.")) or ".blocks." in name or ".layers." in name):
            out.add(name)
    return out


def _clean(name):
    """Parameter name without the prefixes that sharding / data-parallel wrappers insert."""
    name = name.replace("_fsdp_wrapped_module.", "")
    return name[len("module."):] if name.startswith("module.") else name


def build_optimizer(lib, cfg, model, mat_names):
    mats, rest = [], []
    for name, p in model.named_parameters():
        if p.requires_grad:
            (mats if _clean(name) in mat_names else rest).append(p)
    kind = cfg["optimizer"]
    if kind == "muon+adamw":
        return lib.SplitOpt([
            {"params": mats, "optimizer": lib.Muon, "lr": 0.02},
            {"params": rest, "optimizer": lib.AdamW, "lr": 3e-4},
        ])
    if kind == "muon-ecc+adamw":
        return lib.SplitOpt([
            {"params": mats, "optimizer": lib.Muon, "lr": 0.02, "ecc": "bf16+8", "param_ecc": "bf16+8", "mars": True,
             "caution": True},
            {"params": rest, "optimizer": lib.AdamW, "lr": 3e-4},
        ])  # fmt: skip
    if kind == "psgd":
        return lib.PSGDKron(mats + rest, preconditioner_update_probability=0.1, max_size_triangular=8192, ecc="bf16+8")
    if kind == "soap":
        return lib.SOAP(mats + rest, lr=3e-3, betas=(0.95, 0.95), shampoo_beta=0.95, precondition_frequency=10,
                        max_precond_dim=4096)  # fmt: skip
    raise ValueError(kind)


def roofline_of(cfg, model, opt_ms, world):
    """Fraction of the hardware floor for the optimizer step (only for the Muon + AdamW configurations, whose work
    model is simple enough to state: Newton-Schulz FLOPs plus element-wise bytes)."""
    if not cfg["optimizer"].startswith("muon"):
        return None
    from heavyball_b200.utils import roofline

    names = matrix_names(model)
    shapes, other = [], 0
    for name, p in model.named_parameters():
        if _clean(name) in names and p.ndim >= 2:
            shapes.append(tuple(p.shape))
        else:
            other += p.numel()
    return {"opt_step": roofline.muon_adamw_step(shapes, other, opt_ms, world=world)}


# ---------------------------------------------------------------------------------------- one configuration


def run_config(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    cfg = CONFIGS[args.config]
    torch.manual_seed(0)
    ours = args.impl == "ours"
    model_kind = args.model if ours else "plain"
    model_dtype = torch.bfloat16 if cfg["master"] == "bf16" else None
    autocast = cfg["master"] != "bf16"
    launches = None
    compile_note = None
    if ours:
        import heavyball_b200 as lib
        from heavyball_b200 import ops

        launches = ops.launch_counter
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import heavyball as lib

        mode = args.reference_compile_mode
        if mode is None:
            mode = os.environ.get("HB_REF_COMPILE_MODE")  # unset = the reference's stock setting
        if mode is not None:
            lib.utils.compile_mode = None if mode.lower() in ("", "none") else mode
            compile_note = f"compile_mode={lib.utils.compile_mode!r}"
        else:
            compile_note = f"stock compile_mode={lib.utils.compile_mode!r}"

    model = build_model(cfg, model_kind, device, model_dtype)
    mat_names = matrix_names(model)
    n_params = sum(p.numel() for p in model.parameters())
    sharded = cfg["parallelism"] == "fsdp" and world > 1
    parallel_note = "none"
    if sharded:
        if ours:
            from heavyball_b200.parallel import fsdp as hb_fsdp

            train_model = hb_fsdp.shard(model)
            parallel_note = "fully_shard (FSDP2, DTensor parameters), owner-rank repartition inside the optimizer"
        else:
            from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
            from torch.distributed.fsdp.wrap import ModuleWrapPolicy

            layer_cls = {type(m) for m in (getattr(model, "layers", None) or getattr(model, "blocks"))}
            train_model = FSDP(model, use_orig_params=True, auto_wrap_policy=ModuleWrapPolicy(layer_cls), device_id=local)
            parallel_note = "FullyShardedDataParallel(use_orig_params=True) (FSDP1: the reference's documented path)"
        opt = build_optimizer(lib, cfg, train_model, mat_names)
    else:
        opt = build_optimizer(lib, cfg, model, mat_names)
        if world > 1:
            if ours:
                from heavyball_b200.parallel import ddp as hb_ddp

                mode, why = args.ddp_mode, ""
                try:
                    train_model = hb_ddp.wrap(model, opt, mode=mode)
                except Exception as err:  # noqa: BLE001  (e.g. no symmetric memory between these GPUs)
                    if mode != "peer":
                        raise
                    train_model, why = None, f"{type(err).__name__}: {str(err)[:200]}"
                agreed = torch.tensor([0 if train_model is None else 1], device=device)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                if int(agreed.item()) == 0:
                    if train_model is not None:
                        raise RuntimeError("peer data parallelism came up on this rank but not on all ranks")
                    mode = "nccl"
                    train_model = hb_ddp.wrap(model, opt, mode=mode)
                parallel_note = f"data parallel, gradient path {mode}" + (f" (peer path unavailable: {why})" if why else "")
                ctx = getattr(opt, "_peer", None) or next((getattr(o, "_peer", None) for o in getattr(opt, "optimizers", [])), None)
                if ctx is not None:
                    parallel_note += ", NVSwitch multimem reduce / broadcast" if ctx.multicast else ", per-rank peer loads / stores"
            else:
                from torch.nn.parallel import DistributedDataParallel

                train_model = DistributedDataParallel(model, device_ids=[local])
                parallel_note = "DistributedDataParallel (NCCL all-reduce)"
        else:
            train_model = model

    B, T, V = cfg["seqs_per_gpu"], cfg["seq_len"], cfg["vocab_size"]
    n_host = 8
    gen = torch.Generator().manual_seed(1234 + rank)
    host_tokens = [torch.randint(0, V, (B, T + 1), generator=gen).pin_memory() for _ in range(n_host)]
    dev_tokens = [t.to(device) for t in host_tokens]

    graphed = False

    def forward_backward(tokens):
        if autocast:
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=not graphed):
                loss = train_model(tokens[:, :-1], tokens[:, 1:])
        else:
            loss = train_model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        return loss

    def train_step(tokens):
        loss = forward_backward(tokens)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    launches_per_step = None
    if ours:
        # two eager steps: create the optimizer state, then count this repository's kernel launches per step (inside
        # CUDA graphs the same kernels run, but the Python-side counter only sees them at capture time)
        train_step(dev_tokens[0])  # first step: state initialisation takes its own path
        launches.reset()
        train_step(dev_tokens[1 % n_host])
        launches_per_step = launches.count
        can_graph = model_kind == "native" and cfg["family"] == "gpt" and not sharded and autocast
        if args.graphs != "off" and can_graph:
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

    # ---- phase 1: device-timed windows of exactly --steps steps, inputs already on the GPU
    if launches is not None:
        launches.reset()
    sampler.begin()
    if args.cuda_profiler:
        torch.cuda.profiler.start()
    peer_contexts = []
    if ours and world > 1:
        peer_contexts = list({id(c): c for c in [getattr(o, "_peer", None) for o in [opt, *getattr(opt, "optimizers", [])]]
                              if c is not None}.values())  # fmt: skip
    window_ms, last, work_ms = [], None, []
    for w in range(max(1, args.windows)):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks = []
        barrier()
        start.record()
        for i in range(args.steps):
            last = train_step(dev_tokens[(w * args.steps + i) % n_host])
            if args.trace_steps:
                marks.append(torch.cuda.Event(enable_timing=True))
                marks[-1].record()
        stop.record()
        barrier()
        window_ms.append(max_over_ranks(start.elapsed_time(stop)))
        # the last step of the window, as it ran in the pipelined loop (launches queued while the GPU was still in the
        # backward pass): device time between the optimizer's two cross-rank barriers
        work_ms += [t for t in (ctx.work_ms() for ctx in peer_contexts) if t is not None]
        if marks:
            per_step = [a.elapsed_time(b) for a, b in zip([start] + marks[:-1], marks)]
            print(f"rank {rank} window {w} step ms: " + " ".join(f"{t:.1f}" for t in per_step), file=sys.stderr)
    last = last.detach().clone()  # under CUDA graphs the returned loss is a static buffer that later replays overwrite
    if args.cuda_profiler:
        torch.cuda.profiler.stop()
    n_launch = launches_per_step * args.steps if launches_per_step is not None else None
    clocks = sampler.stop() if (rank == 0 and not args.no_clocks) else None
    step_ms = statistics.median(window_ms) / args.steps

    # ---- the two halves of a step, device-timed separately (same state, fresh gradients every iteration)
    fb_ms, opt_ms, isolated_work_ms = [], [], []
    e_a, e_b, e_c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for i in range(max(4, min(args.steps, 10))):
        torch.cuda.synchronize()
        e_a.record()
        forward_backward(dev_tokens[i % n_host])
        e_b.record()
        torch.cuda.synchronize()
        e_b.record()
        opt.step()
        e_c.record()
        torch.cuda.synchronize()
        opt.zero_grad(set_to_none=True)
        fb_ms.append(e_a.elapsed_time(e_b))
        opt_ms.append(e_b.elapsed_time(e_c))
        isolated_work_ms += [t for t in (ctx.work_ms() for ctx in peer_contexts) if t is not None]
    opt_step_ms = max_over_ranks(statistics.median(opt_ms))
    opt_work_ms = max_over_ranks(statistics.median(work_ms)) if work_ms else None
    opt_work_isolated_ms = max_over_ranks(statistics.median(isolated_work_ms)) if isolated_work_ms else None
    opt_step_max_ms = max_over_ranks(max(opt_ms))  # preconditioner-refresh steps show up here
    fwd_bwd_ms = max_over_ranks(statistics.median(fb_ms))

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
    if ours:
        from heavyball_b200 import ops

        ops.check_status()
        if hasattr(train_model, "peer"):
            train_model.peer.check()
    out = None
    if rank == 0:
        value = B * T * world / (step_ms * 1e-3)
        sm = (clocks or {}).get("sm_mhz")
        roof = None
        try:
            roof = roofline_of(cfg, model, opt_step_ms, world if ours else 1) if ours else None
        except Exception as err:  # noqa: BLE001
            roof = {"error": f"{type(err).__name__}: {err}"}
        out = {
            "metric": f"train tokens/s ({args.config}, {cfg['optimizer']}); optimizer step ms in 'optimizer_step_ms'",
            "impl": args.impl,
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "windows": len(window_ms),
            "ms_per_step": step_ms,
            "window_ms_per_step": [round(w / args.steps, 4) for w in window_ms],
            "ms_x_sm_mhz": (step_ms * sm) if sm else None,
            "optimizer_step_ms": opt_step_ms,
            # peer data parallelism only: the part of the optimizer step between its two cross-rank barriers (the rest
            # is waiting for the slowest rank's backward pass), sampled in the pipelined loop of phase 1, and the same
            # when the host starts issuing the step only after the GPU has drained (as in the optimizer_step_ms loop)
            "optimizer_work_ms": opt_work_ms,
            "optimizer_work_isolated_ms": opt_work_isolated_ms,
            "optimizer_step_max_ms": opt_step_max_ms,
            "fwd_bwd_ms": fwd_bwd_ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": (value / PUBLISHED_BASELINE) if PUBLISHED_BASELINE else None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "config": {
                "model": args.config, "global_batch": B * world, "seq_len": T,
                "parallelism": f"{cfg['parallelism']}{world}",
                "optimizer": OPTIMIZER_TEXT[cfg["optimizer"]],
                "precision": ("bf16 autocast, fp32 master weights" if autocast else "bf16 parameters and compute"),
                "vocab_rows": vocab_rows(cfg),
                "parameters": n_params,
                "l2": "per-step working set (activations, parameters, optimizer state) exceeds the 126 MB L2",
            },
            # how this arm runs the workload above (the workload itself is identical in both arms)
            "implementation": {
                "parallel_impl": parallel_note,
                "model_impl": ("heavyball_b200.models (own LayerNorm / GELU / head+loss kernels)" if model_kind == "native"
                               else "baseline/ref_model.py (plain torch.nn)"),
                "cuda_graphs": "forward and backward replayed from CUDA graphs, optimizer launched eagerly" if graphed else "none",
                "reference_compile": compile_note,
            },
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": n_launch,
            "roofline": roof,
            "final_loss": float(last.detach()),
        }  # fmt: skip
    if ours and out is not None and cfg["optimizer"] == "soap":
        from heavyball_b200.utils import orthogonal

        out["implementation"]["eigenbasis_qr"] = dict(orthogonal.qr_stats)  # fast factorisation taken / refused
    if world > 1:
        dist.destroy_process_group()
    return out


# ---------------------------------------------------------------------------------------- child runs


_SCRUB = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK",
          "ROLE_WORLD_SIZE", "ROLE_NAME", "MASTER_PORT", "MASTER_ADDR", "TORCHELASTIC_RESTART_COUNT",
          "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING",
          "TORCHELASTIC_ERROR_FILE", "OMP_NUM_THREADS")  # fmt: skip


def child_command(args, config, extra, port):
    # SOAP refreshes its eigenbases every 10th step and PSGD fits on every 10th: a timed window spans one whole period,
    # and the warm-up covers the first two refreshes / fits (the first runs eagerly, the second is captured)
    periodic = CONFIGS[config]["optimizer"] in ("soap", "psgd")
    steps, warmup = (10, 22) if periodic else (args.secondary_steps, 3)
    own = [os.path.join(ROOT, "bench.py"), "--gpus", str(args.gpus), "--steps", str(steps), "--warmup", str(warmup),
           "--windows", "3", "--impl", args.impl, "--config", config, "--secondary", "off", "--ddp-mode", args.ddp_mode,
           *extra]  # fmt: skip
    if args.no_clocks:
        own.append("--no-clocks")
    if args.gpus == 1:
        return [sys.executable, *own]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), *own]  # fmt: skip


def run_child(cmd, timeout):
    """Runs one child benchmark in its own process group; returns its JSON line or a record of why there is none."""
    import signal

    env = {k: v for k, v in os.environ.items() if k not in _SCRUB}
    if "torch.distributed.run" in cmd:
        # a child that runs into its time limit is killed as a group; its ranks' memory is then never bound to an
        # NVSwitch multicast object (plain peer loads / stores and NCCL without in-switch reduction instead)
        env.update(NCCL_NVLS_ENABLE="0", HB200_PEER_MULTIMEM="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    t0 = time.time()
    try:
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=ROOT,
                                start_new_session=True)  # fmt: skip
    except OSError as err:
        return {"unavailable": f"could not start: {err}"}
    try:
        stdout, stderr = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(proc.pid, signal.SIGKILL)  # the group this call created, nothing else
        except OSError:
            pass
        proc.communicate()
        return {"unavailable": f"time limit of {timeout:.0f} s reached", "seconds": round(time.time() - t0, 1)}
    for line in reversed(stdout.strip().splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                rec = json.loads(line)
                rec["seconds"] = round(time.time() - t0, 1)
                return rec
            except ValueError:
                continue
    tail = " | ".join((stderr or "").strip().splitlines()[-3:])[-600:]
    return {"unavailable": f"exit code {proc.returncode}: {tail}", "seconds": round(time.time() - t0, 1)}


def _brief(rec):
    """The fields of a child's line that the parent's line keeps."""
    keep = ("impl", "value", "unit", "n_gpus", "steps", "warmup", "windows", "ms_per_step", "optimizer_step_ms",
            "optimizer_step_max_ms", "optimizer_work_ms", "optimizer_work_isolated_ms", "fwd_bwd_ms", "clocks", "e2e", "gpu_launches", "final_loss", "unavailable",
            "seconds", "config", "implementation", "roofline", "note")  # fmt: skip
    return {k: rec[k] for k in keep if k in rec}


def run_secondaries(args, base_port):
    results, t0 = {}, time.time()
    jobs = []
    if args.impl == "ours":
        jobs.append(("plain_model", args.config, ["--model", "plain", "--steps", str(args.steps), "--windows", "3"]))
    jobs += [(name, name, []) for name in SECONDARY]
    for k, (key, config, extra) in enumerate(jobs):
        left = args.secondary_budget - (time.time() - t0)
        if left < 60:
            results[key] = {"unavailable": "skipped: the time budget for child runs was used up"}
            continue
        limit = min(args.secondary_timeout, left)
        rec = run_child(child_command(args, config, extra, base_port + 11 + k), limit)
        if args.impl == "reference" and "unavailable" in rec and not extra and "time limit" not in rec["unavailable"]:
            # documented fallback of the reference: eager execution (its compile path fails on some optimizers here)
            left = args.secondary_budget - (time.time() - t0)
            if left >= 60:
                retry = run_child(child_command(args, config, ["--reference-compile-mode", "none"], base_port + 31 + k),
                                  min(args.secondary_timeout, left))  # fmt: skip
                retry["note"] = f"stock compile path failed ({rec['unavailable'][:300]}); measured with compile_mode=None"
                rec = retry
        results[key] = _brief(rec)
    return results


def main():
    args = parse()
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "heavyball")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return 0
    rank = int(os.environ.get("RANK", "0"))
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    want_children = args.secondary == "on" or (args.secondary == "auto" and args.config == "gpt2-small")
    try:
        out = run_config(args)
    except Exception as err:  # noqa: BLE001
        if args.secondary != "off" or rank != 0:
            raise
        # a child run reports its failure as a record instead of a traceback only
        import traceback

        traceback.print_exc()
        print(json.dumps({"impl": args.impl, "unavailable": f"{type(err).__name__}: {str(err)[:400]}",
                          "config": {"model": args.config}}))  # fmt: skip
        return 0
    if rank != 0:
        return 0
    if want_children:
        import gc

        import torch

        gc.collect()
        torch.cuda.empty_cache()
        extra = run_secondaries(args, base_port)
        if "plain_model" in extra:
            out["plain_model"] = extra.pop("plain_model")
        out["secondary"] = extra
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
