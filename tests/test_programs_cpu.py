"""The staged SOAP / PSGD programs (bucket-major buffers, adopted batched state, per-bucket matrix stage) against the
PyTorch definitions of the same chains, on CPU with library products.  Trajectories must agree to rounding, the state
must keep the checkpoint layout, and a reloaded checkpoint must continue identically (state is adopted again)."""

import copy

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import lowering

SHAPES = [(12, 8), (12, 8), (8, 8), (16,), (1, 6), (12, 8), (5, 40)]
# SOAP's statistics of a 1 x n matrix gain one rank per step; their null space makes the refreshed eigenbasis (and the
# Adam step taken in it) depend on rounding noise, so the comparison uses shapes whose statistics reach full rank
SOAP_SHAPES = [(12, 8), (12, 8), (8, 8), (16,), (3, 2), (12, 8), (5, 40)]


def _run(name, kwargs, steps, lowered, reload_at=None):
    torch.manual_seed(0)
    shapes = SOAP_SHAPES if name.startswith("SO") else SHAPES
    params = [torch.nn.Parameter(torch.randn(*s) * 0.5) for s in shapes]
    lowering.cpu_programs = lowered
    try:
        torch.manual_seed(1)
        opt = getattr(hb, name)(params, **kwargs)
        g = torch.Generator().manual_seed(5)
        for step in range(steps):
            if reload_at is not None and step == reload_at:
                sd = copy.deepcopy(opt.state_dict())
                opt = getattr(hb, name)(params, **kwargs)
                opt.load_state_dict(sd)
            for p in params:
                p.grad = torch.randn(p.shape, generator=g) * 0.1
            opt.step()
        return [p.detach().clone() for p in params], opt
    finally:
        lowering.cpu_programs = False


CASES = [
    ("SOAP", dict(lr=1e-2, precondition_frequency=2, max_precond_dim=32)),
    ("SOAP", dict(lr=1e-2, precondition_frequency=3, max_precond_dim=10, caution=True)),  # one-sided and no eigenbasis
    ("SOLP", dict(lr=1e-2, precondition_frequency=2, max_precond_dim=32)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=1.0)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=0.5, max_size_triangular=10, caution=True)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=1.0, store_triu_as_line=False, update_clipping=None)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=1.0, mars=True, weight_decay=0.1)),
]


@pytest.mark.parametrize("name,kwargs", CASES, ids=[f"{n}-{i}" for i, (n, _) in enumerate(CASES)])
def test_staged_program_matches_pytorch_definitions(name, kwargs):
    want, ref_opt = _run(name, kwargs, 6, lowered=False)
    got, opt = _run(name, kwargs, 6, lowered=True)
    assert lowering._program(opt) is not None and lowering._program(opt).kind in ("soap", "psgd")
    assert any(k[0] == "bucket" for k in lowering._program(opt).workspace)  # the staged path did run
    for w, g in zip(want, got):
        torch.testing.assert_close(g, w, rtol=2e-4, atol=2e-5)
    # checkpoint layout is unchanged: same keys, same shapes (leading slot dim of 1), same nesting
    a, b = ref_opt.state_dict()["state"], opt.state_dict()["state"]

    def shape_tree(x):
        if isinstance(x, torch.Tensor):
            return tuple(x.shape)
        if isinstance(x, dict):
            return {k: shape_tree(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return type(x)(shape_tree(v) for v in x)
        return x if not isinstance(x, set) else sorted(x)

    assert shape_tree(a) == shape_tree(b)


@pytest.mark.parametrize("name,kwargs", [CASES[0], CASES[3]], ids=["SOAP", "PSGDKron"])
def test_reloaded_checkpoint_continues_identically(name, kwargs):
    straight, _ = _run(name, kwargs, 6, lowered=True)
    resumed, _ = _run(name, kwargs, 6, lowered=True, reload_at=4)
    for s, r in zip(straight, resumed):
        torch.testing.assert_close(r, s, rtol=1e-6, atol=1e-7)


def test_stage_ranges_are_opened_when_tracing_is_on():
    from heavyball_b200.utils import tracing

    tracing.enable(True, record=True)
    tracing.seen.clear()
    try:
        _run("SOAP", CASES[0][1], 4, lowered=True)
        _run("PSGDKron", CASES[3][1], 3, lowered=True)
    finally:
        tracing.enable(False)
    assert {"soap.project", "soap.refresh", "psgd.fit"} <= set(tracing.seen)
    tracing.seen.clear()
    _run("SOAP", CASES[0][1], 3, lowered=True)
    assert not tracing.seen  # off again: nothing recorded, nothing pushed


def test_which_program_runs_each_class():
    """The chain matcher of the kernel lowering, class by class (no GPU needed to match)."""
    import torch

    import heavyball_b200 as hb
    from heavyball_b200 import lowering

    model = torch.nn.Linear(8, 8)
    want = {
        "AdamW": "elementwise(update_by_adam)",
        "LaProp": "elementwise(update_by_laprop)",
        "ADOPT": "elementwise(update_by_adopt)",
        "NAdam": "elementwise(update_by_nadam)",
        "SFAdamW": "elementwise(scale_by_exp_avg_sq) +schedule_free",
        "Muon": "orthogonal(nesterov_ema)",
        "MuonAdamW": "route[orthogonal(nesterov_ema) | elementwise(scale_by_adam)]",
        "SOAP": "soap(adam)",
        "SOLP": "soap(laprop)",
        "SignLaProp": "elementwise(scale_by_laprop) +sign",
        "OrthoLaProp": "elementwise(update_by_laprop) +orthograd",
        "LaPropOrtho": "elementwise(scale_by_laprop) +project",
        "MSAMLaProp": "elementwise(scale_by_exp_avg_sq) +msam",
        "HyperBallAdamW": "route[elementwise(scale_by_exp_avg_sq) +hyperball | elementwise(scale_by_exp_avg_sq)]",
        "SUDSAdamW": "not lowered",
        "Scion": "not lowered",
    }
    for name, text in want.items():
        opt = getattr(hb, name)(model.parameters(), lr=1e-3)
        assert lowering.describe(opt) == text, name
    assert lowering.describe(hb.PSGDKron(model.parameters(), lr=1e-3)).startswith("psgd(")
    clipped = hb.AdamW(model.parameters(), lr=1e-3, gradient_clipping="l2_clip_")
    assert lowering.describe(clipped) == "elementwise(update_by_adam) +grad_clip"
    assert lowering.describe(hb.SignLaProp(model.parameters(), lr=1e-3, gradient_clipping="l2_clip_")) == "not lowered"
