"""Training step with the forward and backward pass replayed from CUDA graphs.

    python examples/graphed_training.py

A GPT-2-shaped model trains with ``SplitOpt(Muon, AdamW)`` under bf16 autocast.  ``graph_forward_backward`` records
``model(inputs, targets)`` and its backward once; afterwards a step is two graph launches, the gradient accumulation
and the optimizer's handful of kernels, instead of roughly 1 500 launches.  Shapes and dtypes must stay as captured.
"""

import time

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb
from heavyball_b200.models import GPT, GPTConfig, graph_forward_backward, split_param_groups


def main():
    torch.manual_seed(0)
    device = torch.device("cuda")
    model = GPT(GPTConfig(n_layer=4, n_head=8, d_model=512, vocab_size=32000, seq_len=512)).to(device)
    matrices, rest = split_param_groups(model)
    opt = hb.SplitOpt([
        {"params": matrices, "optimizer": hb.Muon, "lr": 0.02},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-4},
    ])
    batches = [torch.randint(0, 32000, (8, 513), device=device) for _ in range(4)]

    def step(tokens):
        with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
            loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        return loss

    def timed(n):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n):
            loss = step(batches[i % len(batches)])
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n * 1e3, float(loss)

    step(batches[0])  # creates the optimizer state with ordinary launches
    print("eager   : %.2f ms/step, loss %.3f" % timed(20))
    graph_forward_backward(model, (batches[0][:, :-1], batches[0][:, 1:]))
    print("graphed : %.2f ms/step, loss %.3f" % timed(20))


if __name__ == "__main__":
    main()
