"""Small, self-terminating workloads for kernel profiling (launch lists and single-kernel captures).

    python benchmarks/profile_targets.py opt_step_gpt2   # 3 optimizer steps, GPT-2-small parameter shapes
    python benchmarks/profile_targets.py ns_small        # Newton-Schulz on 8 x (1024 x 4096) bf16-sized work
    python benchmarks/profile_targets.py adam_small      # fused AdamW over 64M fp32 parameters (768 MB state+params)

Each case holds well under a few GB on the device and launches only a handful of kernels.
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import heavyball_b200 as hb  # noqa: E402
from heavyball_b200 import ops, utils  # noqa: E402


def opt_step_gpt2(steps=3):
    from heavyball_b200.models import GPT, GPTConfig, split_param_groups

    m = GPT(GPTConfig(12, 12, 768, 0, 50257, 1024)).cuda()
    mats, rest = split_param_groups(m)
    opt = hb.SplitOpt([
        {"params": mats, "optimizer": hb.Muon, "lr": 0.02},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-4},
    ])
    grads = [torch.randn_like(p) * 0.01 for p in m.parameters()]

    def one_step():
        for p, g in zip(m.parameters(), grads):
            p.grad = g
        opt.step()

    one_step()  # the first step initialises state through the PyTorch path
    one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()  # with `ncu --profile-from-start off` only the steady-state steps are captured
    for _ in range(steps):
        one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def ns_small():
    mats = [torch.randn(1024, 4096, device="cuda") for _ in range(8)]
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()
    print(float(out.abs().mean()))


def adam_small():
    params = [torch.nn.Parameter(torch.randn(4096, 4096, device="cuda")) for _ in range(4)]
    opt = hb.AdamW(params, lr=1e-3, consume_grad=False)
    for p in params:
        p.grad = torch.randn_like(p)
    for _ in range(3):
        opt.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    opt.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


if __name__ == "__main__":
    {"opt_step_gpt2": opt_step_gpt2, "ns_small": ns_small, "adam_small": adam_small}[sys.argv[1]]()
