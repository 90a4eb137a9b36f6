"""A small convolutional autoencoder trained with PSGDPRO on synthetic images (conv kernels are merged into
matrices by ``merge_dims`` before the Kronecker factors are built)."""

import torch
import torch.nn as nn

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb

if __name__ == "__main__":
    torch.manual_seed(0)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = nn.Sequential(
        nn.Conv2d(1, 16, 3, 2, 1), nn.GELU(), nn.Conv2d(16, 32, 3, 2, 1), nn.GELU(),
        nn.ConvTranspose2d(32, 16, 4, 2, 1), nn.GELU(), nn.ConvTranspose2d(16, 1, 4, 2, 1),
    ).to(dev)  # fmt: skip
    opt = hb.PSGDPRO(model.parameters(), lr=1e-3, merge_dims=True, max_size_triangular=256)
    basis = torch.randn(8, 1, 28, 28, device=dev)
    for step in range(200):
        x = torch.einsum("bk,kchw->bchw", torch.randn(64, 8, device=dev), basis)
        loss = nn.functional.mse_loss(model(x), x)
        loss.backward()
        opt.step()
        opt.zero_grad()
        if step % 50 == 0:
            print(step, round(loss.item(), 4))
