"""Composing a new optimizer from transforms: Adam's magnitude grafted onto the raw gradient direction.

``Parallel`` runs several sub-chains on copies of the update and merges their outputs with a user function.
"""

import torch
import torch.nn as nn

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200.chainable as C


def graft(outputs, eps: float = 1e-8):
    adam, sgd = outputs
    return [s * (a.norm() / s.norm().add(eps)) for a, s in zip(adam, sgd)]


class GraftedAdam(C.BaseOpt):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-4, warmup_steps=0):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps)
        branch = C.Parallel(branches=[[C.scale_by_adam], [C.identity]], merge_fn=graft)
        super().__init__(params, defaults, fns=(branch,))


if __name__ == "__main__":
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 4))
    opt = GraftedAdam(model.parameters(), lr=3e-3)
    x, y = torch.randn(512, 32), torch.randint(0, 4, (512,))
    for step in range(200):
        loss = nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        if step % 50 == 0:
            print(step, round(loss.item(), 4))
