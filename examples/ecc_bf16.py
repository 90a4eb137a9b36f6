"""Precision study: optimizer state and parameters in bf16, bf16 + 8-bit error correction, fp32.

Trains the same regression model three ways and prints the final losses and state bytes.  ``ecc="bf16+8"``
stores every state tensor as bf16 plus an int8 residual (3 bytes per element instead of 4) and tracks the
fp32 trajectory closely; plain ``storage_dtype="bfloat16"`` is cheaper (2 bytes) but noisier.
"""

import torch
import torch.nn as nn

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb


def run(**kw):
    torch.manual_seed(0)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = nn.Sequential(nn.Linear(64, 256), nn.Tanh(), nn.Linear(256, 1)).to(dev)
    opt = hb.AdamW(model.parameters(), lr=2e-3, **kw)
    x = torch.randn(2048, 64, device=dev)
    y = x[:, :8].square().sum(1, keepdim=True)
    for _ in range(400):
        loss = nn.functional.mse_loss(model(x.to(next(model.parameters()).dtype)).float(), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
    return loss.item(), opt.state_size()


if __name__ == "__main__":
    for name, kw in [("fp32", {}), ("bf16 state", {"storage_dtype": "bfloat16"}), ("bf16+8 state", {"ecc": "bf16+8"}),
                     ("bf16+8 state and params", {"ecc": "bf16+8", "param_ecc": "bf16+8"})]:
        loss, size = run(**kw)
        print(f"{name:26s} final loss {loss:.5f}   optimizer state {size / 1024:.0f} KiB")
