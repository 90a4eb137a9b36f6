"""Data-parallel training wrapper.

``wrap(model, optimizer)`` returns a module whose backward leaves identical, averaged gradients on
every rank before ``optimizer.step()`` runs.  The collective path is NCCL (``DistributedDataParallel``
with gradient-as-bucket-view); see ``heavyball_b200.parallel.fused_reduce`` for the peer-memory
kernels that replace it on NVLink-connected GPUs.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def wrap(model: torch.nn.Module, optimizer=None, **kwargs):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return model
    from torch.nn.parallel import DistributedDataParallel

    device_ids = [torch.cuda.current_device()] if next(model.parameters()).is_cuda else None
    kwargs.setdefault("gradient_as_bucket_view", True)
    return DistributedDataParallel(model, device_ids=device_ids, **kwargs)
