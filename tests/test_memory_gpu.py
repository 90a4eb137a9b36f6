"""Memory behaviour on the GPU: AdamW's footprint stays within parameters + gradients + two moments, and a long PSGD run
does not grow (modelled on the reference's ``test/test_memory.py:28,73-74`` and ``test/test_memory_leak.py:36``)."""

import pytest
import torch

import heavyball_b200 as hb

pytestmark = pytest.mark.gpu


def _model(width=2048, depth=8):  # 134 MB of parameters: library workspaces (tens of MB) stay small beside it
    torch.manual_seed(0)
    layers = []
    for _ in range(depth):
        layers += [torch.nn.Linear(width, width), torch.nn.Tanh()]
    return torch.nn.Sequential(*layers).cuda()


def test_adamw_peak_memory_envelope():
    model = _model()
    model_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    opt = hb.AdamW(model.parameters(), lr=1e-3)
    x = torch.randn(8, 2048, device="cuda")
    rest = None
    for step in range(6):
        if step == 2:  # state exists, the allocator and the library workspaces are warm, gradients are released
            torch.cuda.synchronize()
            rest = torch.cuda.memory_allocated()
            torch.cuda.reset_peak_memory_stats()
        model(x).square().mean().backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated()
    assert opt.state_size() < 2.05 * model_bytes  # two moments, nothing else of parameter size
    # at rest: parameters + two moments (+ library workspaces); a step adds the gradients and small activations.
    # A parameter-sized temporary in the fused step would show as 2x here.
    assert rest >= 3.0 * model_bytes, (rest / model_bytes)
    assert peak - rest < 1.3 * model_bytes, ((peak - rest) / model_bytes, rest / model_bytes)


def test_long_psgd_run_does_not_grow():
    model = _model(width=256, depth=3)
    opt = hb.PSGDKron(model.parameters(), lr=1e-3, preconditioner_update_probability=0.5)
    x = torch.randn(16, 256, device="cuda")
    marks = {}
    for step in range(1, 501):
        model(x).square().mean().backward()
        opt.step()
        opt.zero_grad()
        if step in (100, 500):
            torch.cuda.synchronize()
            marks[step] = (torch.cuda.memory_allocated(), torch.cuda.max_memory_allocated())
            torch.cuda.reset_peak_memory_stats()
    assert marks[500][0] <= 1.10 * marks[100][0], marks
    assert marks[500][1] <= 1.10 * max(marks[100][1], 1), marks
    hb.ops.check_status()
