"""CUDA-graph capture of a model's forward and backward pass.

A 12-layer transformer step is about 1 500 kernel launches; on one GPU the host keeps just ahead of the device,
with eight training processes sharing a host it no longer does.  ``graph_forward_backward`` records the forward
pass and the backward pass of ``model(*example_inputs)`` once (``torch.cuda.make_graphed_callables``) and replays
them: two graph launches plus the per-parameter gradient accumulation and the optimizer's few launches per step.
Shapes, dtypes and the autocast state must stay as captured; the optimizer step stays outside the graphs (its
scalar arguments - step count, learning rate, debiasing - change every step).
"""

from __future__ import annotations

import torch


def graph_forward_backward(model: torch.nn.Module, example_inputs: tuple, autocast_dtype=torch.bfloat16, warmup: int = 3):
    """Returns ``model`` with its forward (and the matching backward) replaced by CUDA-graph replays.

    ``example_inputs``: tensors shaped like every later call's arguments.  Call the result under
    ``torch.autocast("cuda", dtype=autocast_dtype, cache_enabled=False)`` - capture runs under the same context,
    and the autocast weight cache must stay off because cached casts would not be replayed.  The value returned
    by a call (the loss) is a static buffer that the next call overwrites: copy it if it must outlive the step."""
    if not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
        raise ValueError("graph capture needs CUDA tensors as example inputs")
    # the capture keeps its sample arguments as the graphs' static input buffers: give it private copies, so that
    # later calls never write into the caller's tensors (nor into views that overlap each other)
    static_inputs = tuple(t.detach().clone() for t in example_inputs)
    with torch.autocast("cuda", dtype=autocast_dtype, cache_enabled=False):
        return torch.cuda.make_graphed_callables(model, static_inputs, num_warmup_iters=warmup)
