"""Editing an existing optimizer's chain after construction: SOAP followed by orthogonalisation.

Assign a new sequence to ``opt.fns`` (do not mutate it in place): the setter re-numbers the new transforms
while keeping the indices - and therefore the checkpoint keys - of the existing ones.
"""

import torch
import torch.nn as nn

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # run from a checkout
import heavyball_b200 as hb

if __name__ == "__main__":
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 64), nn.ReLU(), nn.Linear(64, 1))
    opt = hb.SOAP(model.parameters(), lr=1e-3, precondition_frequency=1)
    opt.fns = (*opt.fns, hb.chainable.orthogonalize_update)
    for step in range(300):
        x = torch.randn(256, 16)

        def closure():
            loss = nn.functional.mse_loss(model(x), x.square().mean(1, keepdim=True))
            loss.backward()
            return loss

        loss = opt.step(closure)
        opt.zero_grad()
        if step % 100 == 0:
            print(step, round(float(loss), 4))
